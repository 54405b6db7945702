"""Compiles the CUDA sources of ``csrc/`` for sm_100a (and the C++ host sources of ``csrc/host/``) into shared
libraries, at first use.

Each library is built with ``nvcc`` directly (no framework headers, so a file compiles in
seconds) into ``marin_b200/csrc/_build/`` beside the sources, named by a hash of its sources
and flags, and loaded with ``ctypes``.  The reference compiles its kernels at start-up too
(NVRTC, crates/cuda/src/gpu.rs:159-164).  If the package folder is read-only the build goes to
a per-user temporary folder.  A line is printed when a compile starts and every few seconds
while it runs, so that a first call does not look hung.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from typing import Dict, List, Optional, Sequence

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class KernelBuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for cand in (os.environ.get("MARIN_B200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise KernelBuildError("nvcc was not found (looked at $MARIN_B200_NVCC, PATH and /usr/local/cuda/bin); "
                           "the CUDA kernels of marin_b200 cannot be built and there is no other path")


HOST_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden"]


def _host_compiler() -> str:
    for cand in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"), shutil.which("clang++")):
        if cand and (os.path.exists(cand) or shutil.which(cand)):
            return cand
    raise KernelBuildError("no C++ compiler was found (looked at $CXX, g++, c++, clang++): the host code of marin_b200 cannot be built")


def _is_host(sources: Sequence[str]) -> bool:
    return all(s.endswith(".cpp") for s in sources)


_build_dir_cache: Optional[str] = None
_dir_lock = threading.Lock()


def _build_dir() -> str:
    global _build_dir_cache
    with _dir_lock:
        if _build_dir_cache is not None:
            return _build_dir_cache
        override = os.environ.get("MARIN_B200_BUILD_DIR")
        candidates = [override] if override else []
        candidates.append(os.path.join(CSRC, "_build"))
        candidates.append(os.path.join(tempfile.gettempdir(), f"marin_b200_build_{os.getuid()}"))
        for path in candidates:
            try:
                os.makedirs(path, exist_ok=True)
                fd, probe = tempfile.mkstemp(prefix=".probe", dir=path)
                os.close(fd)
                os.remove(probe)
                _build_dir_cache = path
                return path
            except OSError:
                continue
        raise KernelBuildError(f"no writable build folder among {candidates}")


def _digest(sources: Sequence[str], flags: Sequence[str]) -> str:
    h = hashlib.sha256()
    folders = sorted({""} | {os.path.dirname(s) for s in sources})       # headers beside the sources count too
    for folder in folders:
        for name in sorted(os.listdir(os.path.join(CSRC, folder))):
            if name.endswith((".cuh", ".h")):
                with open(os.path.join(CSRC, folder, name), "rb") as fh:
                    h.update(os.path.join(folder, name).encode() + b"\0" + fh.read())
    for src in sources:
        with open(os.path.join(CSRC, src), "rb") as fh:
            h.update(src.encode() + b"\0" + fh.read())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:16]


def library_path(name: str, sources: Sequence[str], defines: Sequence[str] = ()) -> str:
    flags = ARCH_FLAGS + BASE_FLAGS + [f"-D{d}" for d in defines]
    return os.path.join(_build_dir(), f"{name}-{_digest(sources, flags)}.so")


def build(name: str, sources: Sequence[str], defines: Sequence[str] = (), verbose: bool = True) -> str:
    """Compiles ``sources`` (names inside csrc/) into one shared library unless it is already built.
    MARIN_B200_DEFINES in the environment (comma separated, e.g. ``DEC_STAGES=2,PDL_WAIT_FIRST``) adds defines to
    every library: the kernels' tuning constants can be overridden for experiments without touching the sources."""
    extra = [x for x in os.environ.get("MARIN_B200_DEFINES", "").split(",") if x]
    host = _is_host(sources)
    flags = (HOST_FLAGS if host else ARCH_FLAGS + BASE_FLAGS) + [f"-D{d}" for d in list(defines) + extra]
    out = os.path.join(_build_dir(), f"{name}-{_digest(sources, flags)}.so")
    if os.path.exists(out):
        return out
    tmp = f"{out}.{os.getpid()}.{threading.get_ident()}.tmp"
    cmd = [_host_compiler() if host else _nvcc()] + flags + ["-I", CSRC, "-o", tmp] + [os.path.join(CSRC, s) for s in sources]
    if verbose:
        print(f"[marin_b200] compiling {name} {'(host code)' if host else 'for sm_100a'} ({', '.join(sources)}) ...", file=sys.stderr, flush=True)
    started = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    while True:
        try:
            output, _ = proc.communicate(timeout=10)
            break
        except subprocess.TimeoutExpired:
            if verbose:
                print(f"[marin_b200] ... still compiling {name} ({time.time() - started:.0f} s)", file=sys.stderr, flush=True)
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise KernelBuildError(f"nvcc failed for {name}:\n{' '.join(cmd)}\n{output}")
    os.replace(tmp, out)
    if verbose:
        print(f"[marin_b200] built {os.path.basename(out)} in {time.time() - started:.1f} s", file=sys.stderr, flush=True)
    return out


def load(name: str, sources: Sequence[str], defines: Sequence[str] = ()) -> ctypes.CDLL:
    """The library, built if need be and loaded once per process."""
    key = name + "|" + "|".join(defines)
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            lib = ctypes.CDLL(build(name, sources, defines))
            _loaded[key] = lib
        return lib


#: every library of the package: name → sources.  ``build_all`` compiles them all.
LIBRARIES: Dict[str, List[str]] = {
    "mb_elementwise": ["elementwise.cu"],
    "mb_gemm_simple": ["gemm_simple.cu"],
    "mb_attention_simple": ["attention_simple.cu"],
    "mb_sampling": ["sampling.cu"],
    "mb_gemm_tc": ["gemm_tc.cu"],
    "mb_host": ["host/cache_core.cpp", "host/scheduler.cpp", "host/sampler.cpp", "host/safetensors.cpp"],
}


#: (head size, query heads per kv head) the fast attention kernels are built for by ``build_all``; any other
#: layout a model brings is compiled when that model first runs
ATTENTION_LAYOUTS = [(128, 4), (128, 5), (128, 2), (16, 2), (32, 4), (48, 2)]


def build_many(jobs: Dict[str, tuple], verbose: bool = True) -> List[str]:
    """Compiles ``{name: (sources, defines)}`` in parallel; returns the libraries' paths."""
    results: Dict[str, object] = {}

    def work(n: str) -> None:
        try:
            results[n] = build(n, jobs[n][0], jobs[n][1], verbose=verbose)
        except Exception as err:  # noqa: BLE001 - reported below
            results[n] = err

    threads = [threading.Thread(target=work, args=(n,)) for n in jobs]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    errors = [r for r in results.values() if isinstance(r, Exception)]
    if errors:
        raise errors[0]
    return [str(results[n]) for n in jobs]


def attention_job(d: int, group: int) -> tuple:
    """Sources and defines of the attention kernels for one head layout."""
    return (["attention_fast.cu"], [f"HEAD_DIM={d}", f"GROUP={group}"])


def attention_tc_job(d: int, group: int) -> tuple:
    """Sources and defines of the tensor-core prefill attention kernel for one head layout."""
    return (["attention_tc.cu"], [f"HEAD_DIM={d}", f"GROUP={group}"])


def build_all(verbose: bool = True) -> List[str]:
    """Compiles every library and the attention kernels for the layouts in ``ATTENTION_LAYOUTS`` (in parallel).
    Used by the build check and before timing."""
    jobs = {n: (src, []) for n, src in LIBRARIES.items()}
    for d, g in ATTENTION_LAYOUTS:
        jobs[f"mb_attention_fast_d{d}_g{g}"] = attention_job(d, g)
        if d in (64, 128):
            jobs[f"mb_attention_tc_d{d}_g{g}"] = attention_tc_job(d, g)
    return build_many(jobs, verbose)


def build_for(model, dtype, verbose: bool = True) -> List[str]:
    """Compiles what this model needs and nothing else: the element-wise and sampling kernels, the matrix products of
    its dtype, and whatever its parts ask for themselves (``Part.kernel_jobs``: attention for its head layouts)."""
    import torch

    jobs = {"mb_elementwise": (LIBRARIES["mb_elementwise"], []), "mb_sampling": (LIBRARIES["mb_sampling"], []),
            "mb_gemm_simple": (LIBRARIES["mb_gemm_simple"], [])}
    if dtype == torch.bfloat16:
        jobs["mb_gemm_tc"] = (LIBRARIES["mb_gemm_tc"], [])
    if hasattr(model, "kernel_jobs"):
        jobs.update(model.kernel_jobs(dtype))
    return build_many(jobs, verbose)
