"""The kernels as Python functions over torch CUDA tensors.

Every function checks shapes and dtypes on the host, then launches hand-written CUDA on the
current stream through ``ctypes``; results land in the ``out`` argument.  There is no other
implementation behind these names: on a machine without CUDA, or if a library cannot be built,
the call raises.  (The reference funnels its launches through checked wrappers the same way,
crates/cuda/src/ops.rs:53-236.)
"""
from __future__ import annotations

import ctypes
import os
import weakref
from typing import Optional

import torch

from . import build

_c_int, _c_float, _c_void_p, _c_size_t = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_size_t

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}

_ERRORS = {-2: "unsupported dtype combination", -3: "unsupported size", -4: "a device-side wait gave up"}


class KernelError(RuntimeError):
    pass


def _code(t: torch.Tensor) -> int:
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} is not supported by the kernels (float32 or bfloat16)") from None


def _ptr(t: Optional[torch.Tensor]):
    return _c_void_p(t.data_ptr()) if t is not None else _c_void_p(0)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current stream's handle (asked of torch on every launch: streams change under graph capture)."""
    if _raw_stream is not None:
        return _c_void_p(_raw_stream(torch.cuda.current_device()))
    return _c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("marin_b200 kernels run on CUDA tensors only; there is no CPU path")
        if t is not None and not t.is_contiguous():
            raise KernelError("marin_b200 kernels need contiguous tensors")


#: how many kernels of this package were launched (a launcher that returned 0 launched one kernel)
launches = 0


def launches_extra(n: int) -> None:
    """A launcher that started more than one kernel says so here."""
    global launches
    launches += n


#: While this is a list, every launch appends what it was and what it had to move and compute (``engine/profile.py``
#: reads it: the stages of a step with their bytes and flops, in launch order).  ``stage_name`` is set by the parts
#: before their calls ("qkv", "attention", "o", ...) and names the launches that follow.
launch_log: Optional[list] = None
stage_name = ""
_pending_cost: Optional[dict] = None


def _cost(nbytes: float = 0, flops: float = 0.0, bytes_per_key: float = 0, flops_per_pair: float = 0.0) -> None:
    """What the next launch has to read and write (bytes) and compute (flops), as the algorithm needs it: every input
    and output once.  Attention's share that grows with the cache is given per cached key read and per (query, key)
    pair, because a captured graph is replayed at other lengths than it was captured at."""
    global _pending_cost
    if launch_log is not None:
        _pending_cost = {"bytes": float(nbytes), "flops": float(flops), "bytes_per_key": float(bytes_per_key),
                         "flops_per_pair": float(flops_per_pair)}


def _size(t) -> int:
    return t.numel() * t.element_size()


def _check(rc: int, what: str) -> None:
    global launches, _pending_cost
    if rc == 0:
        launches += 1
        if launch_log is not None:
            entry = _pending_cost or {"bytes": 0.0, "flops": 0.0, "bytes_per_key": 0.0, "flops_per_pair": 0.0}
            entry["stage"], entry["kernel"] = stage_name, what
            launch_log.append(entry)
            _pending_cost = None
        return
    if rc in _ERRORS:
        raise KernelError(f"{what}: {_ERRORS[rc]}")
    raise KernelError(f"{what}: CUDA error {rc} ({torch.cuda.cudart().cudaGetErrorString(rc) if hasattr(torch.cuda.cudart(), 'cudaGetErrorString') else ''})")


def _lib(name: str):
    return build.load(name, build.LIBRARIES[name])


def embed(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> None:
    _need_cuda(ids, table, out)
    T, h = out.shape
    assert ids.dtype == torch.int32 and ids.numel() == T and table.shape[1] == h and out.dtype == torch.float32
    _cost(T * h * table.element_size() + _size(out) + _size(ids))
    _check(_lib("mb_elementwise").mb_embed(_ptr(ids), _ptr(table), _code(table), _ptr(out), _c_int(T), _c_int(h), _stream()), "embed")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, unit_offset: bool = False) -> None:
    _need_cuda(x, weight, out)
    rows, n = x.shape
    assert x.dtype == torch.float32 and weight.dtype == torch.float32 and weight.numel() == n and out.shape == x.shape
    _cost(_size(x) + _size(out) + _size(weight), 4.0 * rows * n)
    _check(_lib("mb_elementwise").mb_rmsnorm(_ptr(x), _ptr(weight), _c_float(eps), _c_int(int(unit_offset)), _ptr(out),
                                            _code(out), _c_int(rows), _c_int(n), _stream()), "rmsnorm")


#: bf16 products go to the tcgen05 kernel when their shape allows (False: always the plain kernel)
use_tensor_cores = True
#: with few tokens an RMS norm rides on the products around it instead of running as a kernel of its own
couple_norms = True
#: the same with many tokens, in the persistent kernel.  Off: measured on B200 at 2,048 tokens (Qwen3-4B layers) the
#: per-token factors that every tile's epilogue has to gather cost the gate/up product 39 us where the norm's own
#: kernel costs 7.
couple_norms_in_prefill = False
SM_COUNT = 148


class NonFiniteLogits(KernelError):
    """Logits that are NaN or infinite among the values a token may be chosen from; the sampling kernels give such
    rows the id -1 (the reference refuses them: crates/sampler/src/lib.rs:135-137, crates/model/src/qwen3/model.rs:128)."""


class Scratch:
    """Device memory the kernels use besides their inputs and outputs, for ONE stream of work at a time: an engine
    owns one (``Runner.scratch``) and makes it current around its steps (``using``), so that two engines in one
    process, each on a stream of its own, never share a counter or a flag.  Calls outside any ``using`` block
    take a default per device.

    ``error``        one int: the code a kernel leaves when a bounded wait gives up (zero otherwise);
    ``report``       four ints, of which a sampling kernel fills the first with a copy of ``error`` when that is not
                     zero; the sampled ids of a step lie right behind it (``ids``), so that one copy brings both
                     to the host (``read``) and every step learns of a wait that gave up without a wait of its own;
    ``sumsq``        per-token sums of squares that ride from one product to the next (coupled norms);
    ``parked``, ``parked_flags``  stream-K: the partial tile each CTA may park, and a flag per epilogue warp;
    ``argmax_keys``, ``argmax_count``  arg-max over several blocks per row; zero between launches;
    decode attention's partial results grow on demand (``decode_buffers``) unless a captured graph brings its own.
    """

    ARGMAX_ROWS = 4096
    RESULT_ROWS = 4096

    def __init__(self, device):
        global SM_COUNT
        self.device = torch.device(device)
        SM_COUNT = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.sm_count = SM_COUNT
        i32, f32 = dict(device=self.device, dtype=torch.int32), dict(device=self.device, dtype=torch.float32)
        self.error = torch.zeros(1, **i32)
        self.result = torch.zeros(4 + self.RESULT_ROWS, **i32)      # the report, then the sampled ids: one copy reads both
        self.report = self.result[:4]
        self.sumsq = torch.empty(1 << 22, **f32)
        self.parked = torch.empty(self.sm_count * 256 * 128, **f32)
        self.parked_flags = torch.zeros(self.sm_count * 8, **i32)
        self.argmax_keys = torch.zeros(self.ARGMAX_ROWS, device=self.device, dtype=torch.int64)
        self.argmax_count = torch.zeros(self.ARGMAX_ROWS, **i32)
        self._decode = None
        _all_scratch.add(self)

    def decode_buffers(self, requests: int, H: int, K: int, chunks: int, d: int):
        """Partial accumulators, partial (max, sum) and arrival counters of the split-KV decode kernel, at least as
        large as this call needs; they only ever grow, so layers of different head layouts share them."""
        need = requests * H * chunks
        sizes = (need * d, need * 2, requests * K)
        held = self._decode
        if held is None or any(t.numel() < n for t, n in zip(held, sizes)):
            sizes = tuple(max(n, t.numel()) for t, n in zip(held, sizes)) if held is not None else sizes
            held = (torch.empty(sizes[0], device=self.device, dtype=torch.float32),
                    torch.empty(sizes[1], device=self.device, dtype=torch.float32),
                    torch.zeros(sizes[2], device=self.device, dtype=torch.int32))
            self._decode = held
        return held

    def ids(self, rows: int) -> torch.Tensor:
        """Where a step's sampled ids go (int32 ``[rows]``), right behind the report."""
        if rows > self.RESULT_ROWS:
            raise KernelError(f"{rows} rows are sampled in one step; the result buffer holds {self.RESULT_ROWS}")
        return self.result[4:4 + rows]

    def read(self, rows: int):
        """The ids of ``ids(rows)`` as host ints (-1: that row's logits were not finite), read together with the
        report (one copy, one wait): raises ``KernelError`` if a kernel's wait gave up."""
        both = self.result[:4 + rows].tolist()
        if both[0]:
            self.clear()
            raise KernelError(f"a tensor-core kernel's wait on an mbarrier gave up (code {both[0]})")
        return both[4:]

    def check(self) -> None:
        """Raises if a kernel's bounded wait gave up since the last check (reads one int: synchronises)."""
        code = int(self.error.item())
        if code != 0:
            self.clear()
            raise KernelError(f"a tensor-core kernel's wait on an mbarrier gave up (code {code})")

    def clear(self) -> None:
        """After an error: a kernel that gave up may have left its counters and flags set."""
        self.error.zero_()
        self.report.zero_()
        self.parked_flags.zero_()
        self.argmax_keys.zero_()
        self.argmax_count.zero_()
        if self._decode is not None:
            self._decode[2].zero_()


_default_scratch = {}
_all_scratch = weakref.WeakSet()
_current_scratch: Optional[Scratch] = None


def _scratch_for(device) -> Scratch:
    if _current_scratch is not None and _current_scratch.device == device:
        return _current_scratch
    key = (device.type, device.index)
    s = _default_scratch.get(key)
    if s is None:
        s = _default_scratch[key] = Scratch(device)
    return s


class using:
    """``with ops.using(scratch): ...`` — the kernels launched inside take their scratch memory from ``scratch``."""

    def __init__(self, scratch: Optional[Scratch]):
        self.scratch = scratch

    def __enter__(self):
        global _current_scratch
        self.before, _current_scratch = _current_scratch, self.scratch
        return self.scratch

    def __exit__(self, *exc):
        global _current_scratch
        _current_scratch = self.before
        return False


def check_device_errors(device=None) -> None:
    """Raises if a kernel's bounded wait gave up since the last check, under any scratch of this process (on
    ``device`` if one is given).  Reads one int per scratch: synchronises."""
    for s in list(_all_scratch):
        if device is None or s.device == torch.device(device):
            s.check()


def gemm_plan(T: int, N: int, K: int):
    """Tokens per CTA and the number of K slices (1, 2, 4 or 8: the CTAs of one cluster) for the tensor-core
    kernel.  K is cut when there are fewer tiles than SMs, as far as every slice keeps at least 4 k-blocks."""
    bn = 16 if T <= 16 else 32 if T <= 32 else 64 if T <= 64 else 128
    tiles = -(-N // 128) * -(-T // bn)
    nkb = -(-K // 64)
    splits = 1
    if tiles < SM_COUNT:
        for cand in (8, 4, 2):
            per = -(-nkb // cand)
            if tiles * cand <= 2 * SM_COUNT + 32 and per >= 4 and (cand - 1) * per < nkb:
                splits = cand
                break
    return bn, splits


PERSISTENT_TILES = (128, 144, 160, 176, 192, 208, 224, 240, 256)
STREAM_K_TILES = (128, 192, 256)


def persistent_plan(T: int, N: int) -> int:
    """Tokens per tile for the persistent kernel: the tile width whose rounds over the SMs waste the least.
    A tile's time grows with its width plus a fixed part (ramp-up of the ring, the epilogue's tail)."""
    return _tile_by_tile(T, N)[1]


def _tile_by_tile(T: int, N: int):
    best = None
    for bn in PERSISTENT_TILES:
        tiles = -(-N // 128) * -(-T // bn)
        cost = -(-tiles // SM_COUNT) * (bn + 24)
        if best is None or cost < best[0]:
            best = (cost, bn)
    return best


def many_tokens(T: int, N: int, with_heads: bool = False) -> bool:
    """Whether a product of T tokens and N weight rows goes to the persistent kernel (else: one CTA per tile, K cut
    over the CTAs of a cluster where tiles are few).  It needs a round of tiles to be worth it: with fewer tiles than SMs
    the clusters' many CTAs ask for more at once (measured at Qwen3-4B sizes: the down product at 512 tokens 43 us
    against 52, at 768 tokens 45 against 53; o at 768 tokens 23 against 26).  The q|k|v product that finishes its heads
    stays persistent from half a round on: beyond 128 tokens only that kernel can finish them (17.6 us at 256 tokens
    against 18.2 plus the q/k kernel)."""
    tiles = -(-N // 128) * -(-T // 128)
    return T > 128 and tiles >= (SM_COUNT // 2 if with_heads else SM_COUNT)


#: the persistent kernel deals k-blocks instead of tiles over the SMs where whole tiles would leave SMs idle
stream_k = True


#: Stream-K against tile by tile, fitted to timings on B200 (2,048 and 1,024 tokens, layer sizes of 4B to 14B models):
#: a k-block of a 128 x bn tile costs about bn + 138 (the weight tile is fetched whatever the width), and stream-K
#: pays a fixed part worth 7,700 such units (about 8 us: every CTA parks a partial tile at the start and the last
#: epilogue, which nothing overlaps, is longer).  Measured times came out up to 0.1 above the predicted ratio, hence
#: the margin.  Groups walk different k at the same time, so x has to stay in L2 (at 71 MB stream-K lost 6 % where
#: the fit promised 9 %), and with fewer than four token tiles the fit did not hold (0.98 and 1.07 for 0.75 and 0.91).
_KBLOCK_FIXED, _STREAM_K_FIXED, _STREAM_K_MARGIN, _STREAM_K_MAX_X_BYTES = 138, 7700, 0.87, 48 << 20


def stream_k_plan(T: int, N: int, K: int) -> Optional[int]:
    """Tokens per tile if the product should run stream-K, else None.  The CTAs form groups, one CTA per token tile,
    and every group gets the same number of k-blocks of the weight-row tiles laid end to end: the time goes with
    row tiles / groups, without rounding up to whole rounds of tiles.  It needs at least one row tile per group."""
    if not stream_k:
        return None
    best = None
    rows, nkb = -(-N // 128), -(-K // 64)
    for bn in STREAM_K_TILES:
        across = -(-T // bn)
        if across > SM_COUNT or rows < SM_COUNT // across or (_STREAM_K_FIXED > 0 and (across < 4 or T * K * 2 > _STREAM_K_MAX_X_BYTES)):
            continue
        cost = rows / (SM_COUNT // across) * nkb * (bn + _KBLOCK_FIXED) + _STREAM_K_FIXED
        if best is None or cost <= best[0]:
            best = (cost, bn)
    if best is None:
        return None
    bn = persistent_plan(T, N)
    whole = -(-(rows * -(-T // bn)) // SM_COUNT) * nkb * (bn + _KBLOCK_FIXED)
    return best[1] if best[0] < _STREAM_K_MARGIN * whole else None


def _persistent_product(x, w, out, mode: int, T: int, N: int, K: int, s, what: str) -> None:
    lib = _lib("mb_gemm_tc")
    bn = stream_k_plan(T, N, K)
    if bn is not None:
        _check(lib.mb_gemm_tc_persistent_streamk(
            _ptr(x), _ptr(w), _ptr(out), _c_int(mode), _c_int(T), _c_int(N), _c_int(K), _c_int(bn), _c_int(SM_COUNT),
            _ptr(s.parked), ctypes.c_longlong(s.parked.numel()), _ptr(s.parked_flags), _ptr(s.error), _stream()),
            what + ", stream-K")
        return
    _check(lib.mb_gemm_tc_persistent(_ptr(x), _ptr(w), _ptr(out), _c_int(mode), _c_int(T), _c_int(N), _c_int(K),
                                     _c_int(persistent_plan(T, N)), _c_int(SM_COUNT), _ptr(s.error), _stream()), what)


class NormOut:
    """An RMS norm that may ride on a ``+=`` product: ``rows`` (activation dtype ``[T, N]``) is where the normed
    rows are wanted, ``weight`` float32 ``[N]``."""
    __slots__ = ("weight", "unit_offset", "eps", "rows")

    def __init__(self, weight: torch.Tensor, unit_offset: bool, eps: float, rows: torch.Tensor):
        self.weight, self.unit_offset, self.eps, self.rows = weight, bool(unit_offset), float(eps), rows


class NormedRows:
    """The input of a product whose RMS norm is half done: ``rows`` holds ``bf16(h * g)`` (g the norm's weight) and
    ``sumsq[slot, t]`` sums of squares of ``h[t]`` over disjoint groups of columns.  The product that reads it
    multiplies token ``t`` of its result by ``1 / sqrt(sum_slots sumsq[:, t] / dim + eps)``: the same value as
    normalising first, because the factor is one scalar per token.  Only ``gemm`` and ``gemm_swiglu`` read it."""
    __slots__ = ("rows", "sumsq", "slots", "dim", "eps")

    def __init__(self, rows, sumsq, slots, dim, eps):
        self.rows, self.sumsq, self.slots, self.dim, self.eps = rows, sumsq, slots, dim, eps

    shape = property(lambda self: self.rows.shape)
    dtype = property(lambda self: self.rows.dtype)
    device = property(lambda self: self.rows.device)


#: the most tokens for which a norm rides on the product before it.  The kernel takes up to 64; measured on B200
#: (Qwen3-4B layers) a decode step gains 5 % at 1 token and 3 % at 8, and loses 2 % at 64, where the norm's own
#: kernel is small beside the products.
COUPLED_NORM_MAX_TOKENS = 16


def gemm(x, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False, then_norm: Optional[NormOut] = None):
    """``out[t, n] (+)= sum_k x[t, k] * w[n, k]``.  bfloat16 inputs run on the tensor cores (tcgen05, float32
    accumulate); float32 inputs run on the CUDA cores in true float32.

    ``then_norm`` (with ``accumulate``) asks for the RMS norm of the updated ``out``: if this product can carry it,
    a ``NormedRows`` is returned for the next product to finish; otherwise None, and the caller runs the norm."""
    scaled = x if isinstance(x, NormedRows) else None
    if scaled is not None:
        x = scaled.rows
    _need_cuda(x, w, out)
    T, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and tuple(out.shape) == (T, N), (x.shape, w.shape, out.shape)
    if accumulate and out.dtype != torch.float32:
        raise KernelError("gemm: accumulate needs a float32 output")
    _cost(_size(w) + _size(x) + _size(out) * (2 if accumulate else 1) + (_size(then_norm.rows) if then_norm is not None else 0), 2.0 * T * N * K)
    if (use_tensor_cores and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and K % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and T > 0):
        mode = 2 if accumulate else (0 if out.dtype == torch.bfloat16 else 1)
        if many_tokens(T, N):
            s = _scratch_for(x.device)
            lib = _lib("mb_gemm_tc")
            carried = None
            if (then_norm is not None and accumulate and couple_norms and couple_norms_in_prefill and N % 8 == 0
                    and then_norm.rows.dtype == torch.bfloat16 and then_norm.rows.data_ptr() % 16 == 0):
                slots = int(lib.mb_gemm_tc_norm_slots(_c_int(N), _c_int(1)))
                if slots * T <= s.sumsq.numel():
                    carried = NormedRows(then_norm.rows, s.sumsq, slots, N, then_norm.eps)
            if carried is None and scaled is None:
                _persistent_product(x, w, out, mode, T, N, K, s, "gemm (tensor cores, persistent)")
                return None
            _check(lib.mb_gemm_tc_persistent_coupled(
                _ptr(x), _ptr(w), _ptr(out), _c_int(mode), _c_int(T), _c_int(N), _c_int(K), _c_int(persistent_plan(T, N)), _c_int(SM_COUNT),
                _ptr(then_norm.weight) if carried is not None else None, _c_int(int(then_norm.unit_offset)) if carried is not None else _c_int(0),
                _ptr(carried.rows) if carried is not None else None, _ptr(carried.sumsq) if carried is not None else None,
                _ptr(scaled.sumsq) if scaled is not None else None, _c_int(scaled.slots if scaled is not None else 0),
                _c_int(scaled.dim if scaled is not None else 0), _c_float(scaled.eps if scaled is not None else 0.0),
                _ptr(s.error), _stream()), "gemm (tensor cores, persistent, coupled with a norm)")
            return carried
        bn, splits = gemm_plan(T, N, K)
        s = _scratch_for(x.device)
        lib = _lib("mb_gemm_tc")
        carried = None
        if (then_norm is not None and accumulate and couple_norms and T <= COUPLED_NORM_MAX_TOKENS and N % 8 == 0
                and then_norm.rows.dtype == torch.bfloat16 and then_norm.rows.data_ptr() % 16 == 0):
            slots = int(lib.mb_gemm_tc_norm_slots(_c_int(N), _c_int(splits)))
            if slots * T <= s.sumsq.numel():
                carried = NormedRows(then_norm.rows, s.sumsq, slots, N, then_norm.eps)
        if carried is None and scaled is None:
            _check(lib.mb_gemm_tc_cluster(_ptr(x), _ptr(w), _ptr(out), _c_int(mode), _c_int(T), _c_int(N), _c_int(K),
                                          _c_int(bn), _c_int(splits), _ptr(s.error), _stream()), "gemm (tensor cores)")
            return None
        _check(lib.mb_gemm_tc_coupled(
            _ptr(x), _ptr(w), _ptr(out), _c_int(mode), _c_int(T), _c_int(N), _c_int(K), _c_int(bn), _c_int(splits),
            _ptr(then_norm.weight) if carried is not None else None, _c_int(int(then_norm.unit_offset)) if carried is not None else _c_int(0),
            _ptr(carried.rows) if carried is not None else None, _ptr(carried.sumsq) if carried is not None else None,
            _ptr(scaled.sumsq) if scaled is not None else None, _c_int(scaled.slots if scaled is not None else 0),
            _c_int(scaled.dim if scaled is not None else 0), _c_float(scaled.eps if scaled is not None else 0.0),
            _ptr(s.error), _stream()), "gemm (tensor cores, coupled with a norm)")
        return carried
    assert scaled is None, "rows with a pending norm reach only the tensor-core product"
    _check(_lib("mb_gemm_simple").mb_gemm_simple(_ptr(x), _code(x), _ptr(w), _code(w), _ptr(out), _code(out), _c_int(T),
                                                _c_int(N), _c_int(K), _c_int(int(accumulate)), _stream()), "gemm")
    return None


#: with few tokens the q|k|v product finishes its heads itself (norm, rotation, cache write) where the layout allows
fuse_heads = True
FUSED_HEADS_MAX_TOKENS = 128


#: the same for many tokens, in the persistent kernel's epilogue (tile by tile, no stream-K)
fuse_heads_many_tokens = True


def rope_table(ctx, positions, inv_freq) -> torch.Tensor:
    """cos and sin of ``positions * inv_freq`` for every token of the step, float32 ``[T, 2 * len(inv_freq)]`` (cos
    first), made once per step and position encoding and kept in ``ctx.extras``."""
    key = ("rope_table", inv_freq.data_ptr())
    table = ctx.extras.get(key)
    if table is None:
        T, half = positions.shape[0], inv_freq.shape[0]
        table = ctx.workspace.get(f"rope_table_{len(ctx.extras)}", (T, 2 * half), torch.float32)
        _cost(_size(table), 2.0 * T * half)
        _check(_lib("mb_elementwise").mb_rope_table(_ptr(positions), _ptr(inv_freq), _c_int(half), _ptr(table), _c_int(T), _stream()),
               "rope_table")
        ctx.extras[key] = table
    return table


def gemm_qkv_heads(x, w: torch.Tensor, q_out: torch.Tensor, q_weight, k_weight, eps: float, positions, inv_freq, rotary_dim: int,
                   interleaved: bool, slot_mapping, k_cache, v_cache, H: int, K: int, d: int, write_kv: bool = True, ctx=None) -> bool:
    """The product ``x w^T`` with ``w`` = query, key and value rows (or query rows only), each head normed, rotated
    and stored by the product's own epilogue: queries to ``q_out``, keys and values into the paged caches at
    ``slot_mapping``.  Two kernels do it: the one for up to sixteen tokens computes the angles itself; the persistent
    one for many tokens reads them from the step's table (``rope_table``, which needs ``ctx``).  Returns False,
    having done nothing, where neither applies (heads that are not 128 wide, a partial or interleaved rotation,
    float32, a token count between the two): the caller then runs ``gemm`` and ``qk_norm_rope_write``."""
    scaled = x if isinstance(x, NormedRows) else None
    rows = scaled.rows if scaled is not None else x
    T, Kdim = rows.shape
    N = w.shape[0]
    heads_total = H + 2 * K if write_kv else H
    if not (fuse_heads and use_tensor_cores and rows.is_cuda and rows.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and q_out.dtype == torch.bfloat16 and d == 128 and T > 0 and N == heads_total * d
            and Kdim % 8 == 0 and not interleaved and (inv_freq is None or rotary_dim == d)
            and rows.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and (not write_kv or k_cache.dtype == torch.bfloat16)):
        return False
    page_size = k_cache.shape[2] if write_kv else 0
    if T > FUSED_HEADS_MAX_TOKENS:
        if not (fuse_heads_many_tokens and scaled is None and many_tokens(T, N, with_heads=True)
                and (inv_freq is None or ctx is not None)):
            return False
        _need_cuda(rows, w, q_out)
        assert tuple(q_out.shape) == (T, H * d) and w.shape[1] == Kdim
        table = rope_table(ctx, positions, inv_freq) if inv_freq is not None else None
        _cost(_size(w) + _size(rows) + T * N * 2 + (_size(table) if table is not None else 0), 2.0 * T * N * Kdim)
        s = _scratch_for(rows.device)
        _check(_lib("mb_gemm_tc").mb_gemm_tc_persistent_heads(
            _ptr(rows), _ptr(w), _c_int(T), _c_int(N), _c_int(Kdim), _c_int(persistent_plan(T, N)), _c_int(SM_COUNT), _ptr(q_out),
            _ptr(k_cache) if write_kv else None, _ptr(v_cache) if write_kv else None, _ptr(q_weight), _ptr(k_weight), _c_float(eps),
            _ptr(table), _ptr(slot_mapping) if write_kv else None, _c_int(H), _c_int(K), _c_int(page_size), _ptr(s.error), _stream()),
            "gemm (persistent) with heads finished in the epilogue")
        return True
    bn, splits = gemm_plan(T, N, Kdim)
    if T > bn or splits < 2:
        return False
    _need_cuda(rows, w, q_out)
    assert tuple(q_out.shape) == (T, H * d) and w.shape[1] == Kdim
    _cost(_size(w) + _size(rows) + T * N * 2, 2.0 * T * N * Kdim)
    s = _scratch_for(rows.device)
    _check(_lib("mb_gemm_tc").mb_gemm_tc_heads(
        _ptr(rows), _ptr(w), _c_int(T), _c_int(N), _c_int(Kdim), _c_int(bn), _c_int(splits), _ptr(q_out),
        _ptr(k_cache) if write_kv else None, _ptr(v_cache) if write_kv else None, _ptr(q_weight), _ptr(k_weight), _c_float(eps),
        _ptr(positions), _ptr(inv_freq), _ptr(slot_mapping) if write_kv else None, _c_int(H), _c_int(K), _c_int(page_size),
        _ptr(scaled.sumsq) if scaled is not None else None, _c_int(scaled.slots if scaled is not None else 0),
        _c_int(scaled.dim if scaled is not None else 0), _c_float(scaled.eps if scaled is not None else 0.0),
        _ptr(s.error), _stream()), "gemm with heads finished in the epilogue")
    return True


def qk_norm_rope_write(qkv, q_out, q_weight, k_weight, eps, positions, inv_freq, rotary_dim, interleaved,
                       slot_mapping, k_cache, v_cache, H, K, d, write_kv=True) -> None:
    _need_cuda(qkv, q_out, q_weight, k_weight, positions, inv_freq, slot_mapping, k_cache, v_cache)
    T = qkv.shape[0]
    heads_total = H + 2 * K if write_kv else H
    assert qkv.shape[1] == heads_total * d and tuple(q_out.shape) == (T, H * d) and q_out.dtype == qkv.dtype
    assert k_cache.dtype == qkv.dtype and v_cache.dtype == qkv.dtype
    assert k_cache.shape[1] == K and k_cache.shape[3] == d
    page_size = k_cache.shape[2]
    _cost(2 * _size(qkv), 8.0 * T * heads_total * d)
    _check(_lib("mb_elementwise").mb_qk_norm_rope_write(
        _ptr(qkv), _code(qkv), _ptr(q_out), _ptr(q_weight), _ptr(k_weight), _c_float(eps), _ptr(positions),
        _ptr(inv_freq), _c_int(rotary_dim if inv_freq is not None else 0), _c_int(int(interleaved)), _ptr(slot_mapping),
        _ptr(k_cache), _ptr(v_cache), _c_int(T), _c_int(H), _c_int(K), _c_int(d), _c_int(page_size),
        _c_int(int(write_kv)), _stream()), "qk_norm_rope_write")


#: bf16 attention goes to the tensor-core / split-KV kernels when the head layout allows (False: the plain kernel)
use_fast_attention = True
#: prompt portions go to the tcgen05 attention kernel where it applies (heads of 64 or 128, pages >= 16)
use_tc_attention = True
DECODE_SPLITS = (4096, 2048, 1024, 512, 256, 128, 64)      # keys per CTA the split-KV decode kernel may be given
DECODE_CLUSTER_CHUNKS = 8                                   # most chunks the kernel merges as one cluster (see _attention_lib)
_cluster_asked = set()


def decode_split(requests: int, kv_heads: int, longest: int):
    """Keys per CTA and chunks per sequence for decode attention over sequences of up to ``longest`` keys.

    Up to eight chunks of one (request, kv head), sixteen where the device allows (``DECODE_CLUSTER_CHUNKS``), run as
    one thread-block cluster and merge through distributed shared memory; that is preferred, with chunks as long as still give 256 CTAs (measured on B200 at batch 1, 8 and 64 and
    contexts 1024 and 4096).  A few long sequences would leave most SMs idle that way: they get more chunks, merged
    through scratch memory, as long as still give 128 CTAs."""
    pairs = requests * kv_heads
    best = None
    for split in DECODE_SPLITS:
        chunks = -(-longest // split)
        if chunks > DECODE_CLUSTER_CHUNKS:
            break
        best = (split, chunks)
        if pairs * chunks >= 256:
            break
    if best is not None and (pairs * best[1] >= 128 or best[0] <= 1024):
        # clusters of 3, 5, 6 or 7 CTAs are placed badly (measured: 5 chunks take 36 us where 4 take 26): the grid
        # gets a power of two of chunks, those past the sequences' end have nothing to do and say so to their cluster
        chunks = 1
        while chunks < best[1]:
            chunks *= 2
        return best[0], chunks
    for split in DECODE_SPLITS:
        chunks = -(-longest // split)
        if pairs * chunks >= 128 or split == DECODE_SPLITS[-1]:
            return split, chunks


def _attention_lib(d: int, group: int):
    """The fast attention kernels are compiled for one head size and one group size, at first use.  A library also
    says how many chunks the device lets the decode kernel merge as one cluster (8, or 16 where clusters of a
    non-portable size can be placed): ``decode_split`` plans with the smallest answer so far."""
    global DECODE_CLUSTER_CHUNKS, _cluster_asked
    lib = build.load(f"mb_attention_fast_d{d}_g{group}", *build.attention_job(d, group))
    if (d, group) not in _cluster_asked and torch.cuda.is_available():
        widest = int(lib.mb_attn_decode_max_cluster())
        DECODE_CLUSTER_CHUNKS = widest if not _cluster_asked else min(DECODE_CLUSTER_CHUNKS, widest)
        _cluster_asked.add((d, group))
    return lib


def fast_attention_supported(dtype, H: int, K: int, d: int) -> bool:
    return dtype == torch.bfloat16 and d % 16 == 0 and 16 <= d <= 128 and H % K == 0 and 1 <= H // K <= 8


def decode_scratch(device, requests: int, H: int, K: int, chunks: int, d: int):
    """Scratch of the split-KV decode kernel: partial accumulators, partial (max, sum), and one counter per
    (request, kv head) that is zero between launches."""
    need = requests * H * chunks
    return (torch.empty(need * d, device=device, dtype=torch.float32), torch.empty(need * 2, device=device, dtype=torch.float32),
            torch.zeros(requests * K, device=device, dtype=torch.int32))


class DecodePlan:
    """How single-token attention splits its keys, fixed ahead for a captured graph: keys per CTA, chunks per
    sequence, and scratch memory of the capture's own (partial accumulators, partial (max, sum), counters)."""
    __slots__ = ("split", "chunks", "buffers")

    def __init__(self, split: int, chunks: int, buffers=None):
        self.split, self.chunks, self.buffers = int(split), int(chunks), buffers


def decode_plan(device, dtype, requests: int, H: int, K: int, d: int, span: int) -> Optional[DecodePlan]:
    """The plan for ``requests`` single-token requests over sequences of up to ``span`` keys, with scratch sized for
    exactly this head layout; None where the split-KV kernel does not apply (the plain kernel needs no plan)."""
    if not (use_fast_attention and fast_attention_supported(dtype, H, K, d)):
        return None
    _attention_lib(d, H // K)                        # the library says how wide a cluster may be: plan after asking
    split, chunks = decode_split(requests, K, span)
    return DecodePlan(split, chunks, decode_scratch(device, requests, H, K, chunks, d))


def attention_jobs(dtype, H: int, K: int, d: int) -> dict:
    """``{library: (sources, defines)}`` of the attention kernels a mixer of this head layout runs."""
    if not fast_attention_supported(dtype, H, K, d):
        return {"mb_attention_simple": (build.LIBRARIES["mb_attention_simple"], [])}
    jobs = {f"mb_attention_fast_d{d}_g{H // K}": build.attention_job(d, H // K)}
    if d in (64, 128):
        jobs[f"mb_attention_tc_d{d}_g{H // K}"] = build.attention_tc_job(d, H // K)
    return jobs


def _attention_cost(q, rows: int, H: int, K: int, d: int, which: str) -> None:
    """Queries in, results out; per cached key read, its key and value over all kv heads; per (query, key) pair a
    score and a weighted value for every head.  ``which`` says whose keys and pairs count: the single-token rows'
    ("decode"), the portions' ("prefill") or everyone's ("all")."""
    if launch_log is not None:
        size = q.element_size()
        _cost(2 * rows * H * d * size, 0.0, 2 * K * d * size, 4.0 * H * d)
        _pending_cost["rows"] = which


def attention(q, k_cache, v_cache, out, ctx, block_table, H, K, d, scale, window=0, plan: Optional[DecodePlan] = None) -> None:
    """Causal attention of the step's tokens over the paged cache (their own keys included).  The first
    ``ctx.num_decode`` requests bring one token each (rows 0..num_decode-1); the rest bring portions.  ``plan``
    fixes the split of the single-token rows' keys (a captured graph brings it); without one the split follows the
    longest sequence of the step."""
    _need_cuda(q, k_cache, v_cache, out, block_table)
    T = q.shape[0]
    page_size = k_cache.shape[2]
    assert tuple(q.shape) == (T, H * d) and out.shape == q.shape and k_cache.dtype == q.dtype
    if T == 0:
        return
    if use_fast_attention and fast_attention_supported(q.dtype, H, K, d):
        lib = _attention_lib(d, H // K)
        max_pages = block_table.shape[1]
        nd = ctx.num_decode
        if nd > 0:
            split, chunks = (plan.split, plan.chunks) if plan is not None else decode_split(nd, K, ctx.max_seq_len)
            buffers = plan.buffers if plan is not None and plan.buffers is not None else None
            part_acc, part_ml, counters = buffers or _scratch_for(q.device).decode_buffers(nd, H, K, chunks, d)
            _attention_cost(q, nd, H, K, d, "decode")
            _check(lib.mb_attn_decode(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), _c_int(max_pages),
                                      _ptr(ctx.seq_lens), _c_int(nd), _c_int(K), _c_int(page_size),
                                      ctypes.c_longlong(k_cache.shape[0]), _c_float(scale), _c_int(window), _ptr(part_acc),
                                      _ptr(part_ml), _ptr(counters), _c_int(chunks), _c_int(split),
                                      _ptr(_scratch_for(q.device).error), _stream()), "attention (decode)")
        if ctx.num_requests > nd and use_tc_attention and d in (64, 128) and page_size >= 16:
            tc = build.load(f"mb_attention_tc_d{d}_g{H // K}", *build.attention_tc_job(d, H // K))
            _attention_cost(q, T - nd, H, K, d, "prefill")
            _check(tc.mb_attn_prefill_tc(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), _c_int(max_pages),
                                         _ptr(ctx.cu_tokens), _ptr(ctx.seq_lens), _c_int(nd), _c_int(ctx.num_requests - nd),
                                         _c_int(ctx.max_query_len), _c_int(T), _c_int(K), _c_int(page_size),
                                         ctypes.c_longlong(k_cache.shape[0]), _c_float(scale), _c_int(window),
                                         _ptr(_scratch_for(q.device).error), _stream()), "attention (prefill, tensor cores)")
        elif ctx.num_requests > nd:
            _attention_cost(q, T - nd, H, K, d, "prefill")
            _check(lib.mb_attn_prefill(_ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(block_table), _c_int(max_pages),
                                       _ptr(ctx.cu_tokens), _ptr(ctx.seq_lens), _c_int(nd), _c_int(ctx.num_requests - nd),
                                       _c_int(ctx.max_query_len), _c_int(K), _c_int(page_size), _c_float(scale),
                                       _c_int(window), _stream()), "attention (prefill)")
        return
    _attention_cost(q, T, H, K, d, "all")
    _check(_lib("mb_attention_simple").mb_attention_simple(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _code(q), _ptr(block_table), _c_int(block_table.shape[1]),
        _ptr(ctx.req_index), _ptr(ctx.positions), _c_int(T), _c_int(H), _c_int(K), _c_int(d), _c_int(page_size),
        _c_float(scale), _c_int(window), _stream()), "attention")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> None:
    """``out[t, i] = silu(g) * u``; gate and up are the two halves of a row of ``gate_up``, or (``interleaved``)
    alternate in blocks of 16 columns."""
    _need_cuda(gate_up, out)
    T, I = out.shape
    assert gate_up.shape == (T, 2 * I) and gate_up.dtype == out.dtype and (not interleaved or I % 16 == 0)
    _cost(_size(gate_up) + _size(out), 8.0 * T * I)
    _check(_lib("mb_elementwise").mb_swiglu(_ptr(gate_up), _ptr(out), _code(out), _c_int(T), _c_int(I), _c_int(int(interleaved)),
                                           _stream()), "swiglu")


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """One matrix whose rows alternate 16 gate rows and the 16 up rows of the same indices: the layout the
    fused SwiGLU epilogue of the matrix product reads (``[I, h]`` twice → ``[2 I, h]``; ``I`` a multiple of 16)."""
    I, h = gate.shape
    assert up.shape == gate.shape and I % 16 == 0
    return torch.stack([gate.view(I // 16, 16, h), up.view(I // 16, 16, h)], dim=1).reshape(2 * I, h)


def can_fuse_swiglu(dtype, hidden: int, intermediate: int) -> bool:
    return dtype == torch.bfloat16 and intermediate % 16 == 0 and hidden % 8 == 0


def gemm_swiglu(x: torch.Tensor, w_interleaved: torch.Tensor, out: torch.Tensor, workspace=None) -> None:
    """``out = silu(x Wg^T) * (x Wu^T)`` with ``w_interleaved = interleave_gate_up(Wg, Wu)``: on the tensor cores the
    activation is applied to the float32 accumulators in the epilogue and the ``[T, 2 I]`` intermediate never
    exists; otherwise the product and the activation run as two kernels."""
    scaled = x if isinstance(x, NormedRows) else None
    if scaled is not None:
        x = scaled.rows
    _need_cuda(x, w_interleaved, out)
    T, K = x.shape
    N = w_interleaved.shape[0]
    I = N // 2
    assert tuple(out.shape) == (T, I) and w_interleaved.shape[1] == K and out.dtype == x.dtype
    fused = (use_tensor_cores and x.dtype == torch.bfloat16 and w_interleaved.dtype == torch.bfloat16 and K % 8 == 0
             and N % 32 == 0 and x.data_ptr() % 16 == 0 and w_interleaved.data_ptr() % 16 == 0 and T > 0)
    if not fused:
        tmp = workspace.get("gate_up", (T, N), x.dtype) if workspace is not None else torch.empty(T, N, device=x.device, dtype=x.dtype)
        gemm(scaled if scaled is not None else x, w_interleaved, tmp)
        swiglu(tmp, out, interleaved=True)
        return
    s = _scratch_for(x.device)
    _cost(_size(w_interleaved) + _size(x) + _size(out), 2.0 * T * N * K)
    if many_tokens(T, N):
        if scaled is not None:
            _check(_lib("mb_gemm_tc").mb_gemm_tc_persistent_coupled(
                _ptr(x), _ptr(w_interleaved), _ptr(out), _c_int(3), _c_int(T), _c_int(N), _c_int(K), _c_int(persistent_plan(T, N)),
                _c_int(SM_COUNT), None, _c_int(0), None, None, _ptr(scaled.sumsq), _c_int(scaled.slots), _c_int(scaled.dim),
                _c_float(scaled.eps), _ptr(s.error), _stream()), "gemm+swiglu (tensor cores, persistent, coupled with a norm)")
            return
        _persistent_product(x, w_interleaved, out, 3, T, N, K, s, "gemm+swiglu (tensor cores, persistent)")
        return
    bn, _ = gemm_plan(T, N, K)
    if scaled is not None:
        _check(_lib("mb_gemm_tc").mb_gemm_tc_coupled(
            _ptr(x), _ptr(w_interleaved), _ptr(out), _c_int(3), _c_int(T), _c_int(N), _c_int(K), _c_int(bn), _c_int(1),
            None, _c_int(0), None, None, _ptr(scaled.sumsq), _c_int(scaled.slots), _c_int(scaled.dim), _c_float(scaled.eps),
            _ptr(s.error), _stream()), "gemm+swiglu (tensor cores, coupled with a norm)")
        return
    _check(_lib("mb_gemm_tc").mb_gemm_tc_cluster(_ptr(x), _ptr(w_interleaved), _ptr(out), _c_int(3), _c_int(T), _c_int(N), _c_int(K),
                                                _c_int(bn), _c_int(1), _ptr(s.error), _stream()), "gemm+swiglu (tensor cores)")


def gather_rows(src: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
    _need_cuda(src, rows, out)
    W, h = out.shape
    assert src.dtype == torch.float32 and out.dtype == torch.float32 and rows.dtype == torch.int32 and rows.numel() == W
    _cost(2 * _size(out))
    _check(_lib("mb_elementwise").mb_gather_rows(_ptr(src), _ptr(rows), _ptr(out), _c_int(W), _c_int(h), _stream()), "gather_rows")


def add_into(y: torch.Tensor, x: torch.Tensor) -> None:
    """``y += x`` with ``y`` float32 (the residual stream)."""
    _need_cuda(y, x)
    assert y.dtype == torch.float32 and y.numel() == x.numel()
    _cost(2 * _size(y) + _size(x), float(y.numel()))
    _check(_lib("mb_elementwise").mb_add_into(_ptr(y), _ptr(x), _code(x), _c_size_t(y.numel()), _stream()), "add_into")


def argmax(logits: torch.Tensor, usable: int, out: torch.Tensor, feed: Optional[torch.Tensor] = None,
           mirror: Optional[torch.Tensor] = None, which: Optional[torch.Tensor] = None) -> None:
    """``out[r]`` = id of the largest of the first ``usable`` logits of row ``r`` (lowest id among equals); -1 for a
    row that holds a NaN or an infinity among them.

    ``feed`` (int32 ``[rows]`` on the device) receives the ids too (0 for such a row): the next step's token ids, for a
    step that is launched before the host has seen these.  ``mirror`` (pinned host memory, int32 ``[2, 4 + rows or more]``)
    with ``which`` (a device int, 0 or 1): row ``which`` of it receives the error code of the current scratch, three zeros
    and the ids, written by the kernel itself; the host reads them once an event recorded behind the launch has completed."""
    _need_cuda(logits, out, feed, which)
    rows, vocab = logits.shape
    assert logits.dtype == torch.float32 and out.dtype == torch.int32 and out.numel() == rows
    assert feed is None or (feed.dtype == torch.int32 and feed.numel() >= rows)
    if mirror is not None:
        assert (mirror.dtype == torch.int32 and mirror.is_pinned() and mirror.dim() == 2 and mirror.shape[0] == 2 and mirror.is_contiguous()
                and mirror.shape[1] >= 4 + rows and which is not None and which.dtype == torch.int32 and rows <= _scratch_for(logits.device).ARGMAX_ROWS)
    s = _scratch_for(logits.device)
    _cost(rows * usable * 4)
    _check(_lib("mb_sampling").mb_argmax(_ptr(logits), _c_int(rows), _c_int(vocab), _c_int(usable), _ptr(out), _ptr(s.argmax_keys),
                                        _ptr(s.argmax_count), _c_int(s.ARGMAX_ROWS), _c_int(2 * s.sm_count), _ptr(s.report),
                                        _ptr(s.error), _ptr(feed), _ptr(mirror), _c_int(mirror.shape[1] if mirror is not None else 0),
                                        _ptr(which), _stream()), "argmax")


def sample(logits: torch.Tensor, usable: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           uniform: torch.Tensor, out: torch.Tensor) -> None:
    """Draws one token per row from the reference's kept set (temperature, top-k, top-p; temperature 0 = greedy):
    ``uniform[r]`` in [0, 1) selects the token by walking the kept ids in increasing order.  Rows with a logit that is
    not finite get the id -1."""
    _need_cuda(logits, usable, temperature, top_k, top_p, uniform, out)
    rows, vocab = logits.shape
    assert logits.dtype == torch.float32 and out.dtype == torch.int32 and usable.dtype == torch.int32 and top_k.dtype == torch.int32
    assert temperature.dtype == torch.float32 and top_p.dtype == torch.float32 and uniform.dtype == torch.float32
    assert all(t.numel() == rows for t in (usable, temperature, top_k, top_p, uniform, out))
    s = _scratch_for(logits.device)
    _cost(_size(logits))
    _check(_lib("mb_sampling").mb_sample(_ptr(logits), _c_int(rows), _c_int(vocab), _ptr(usable), _ptr(temperature), _ptr(top_k),
                                        _ptr(top_p), _ptr(uniform), _ptr(out), _ptr(s.report), _ptr(s.error), _stream()), "sample")
