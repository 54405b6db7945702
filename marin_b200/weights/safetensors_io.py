"""Reading and writing the safetensors container.

Layout (the same the reference parses, crates/loader/src/safetensors.rs:54-106):
8 bytes little-endian header length, a JSON header mapping tensor name to
``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the end of
the header), then the raw little-endian tensor bytes.  The file is memory-mapped;
tensors are views until they are copied to the device.
"""
from __future__ import annotations

import ctypes
import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Tuple

import numpy as np
import torch

MAX_HEADER_BYTES = 100 * 1024 * 1024

_DTYPES = {
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "F32": (torch.float32, 4),
    "F64": (torch.float64, 8),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
    "I16": (torch.int16, 2),
    "I32": (torch.int32, 4),
    "I64": (torch.int64, 8),
    "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    """A safetensors file that cannot be trusted: truncated, bad header, bad offsets."""


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    begin: int
    end: int


class SafetensorsFile:
    """One memory-mapped safetensors file."""

    def __init__(self, path: str):
        """The header is read and checked by the C++ host library (``csrc/host/safetensors.cpp``); the bytes are
        mapped here."""
        from ..cache.pages import host_lib

        self.path = path
        lib = host_lib()
        err = ctypes.create_string_buffer(1024)
        handle = lib.mbl_open(os.fsencode(path), err, len(err))
        if not handle:
            raise SafetensorsError(err.value.decode("utf-8", "replace"))
        try:
            self.data_start = int(lib.mbl_data_start(handle))
            self.tensors: Dict[str, TensorInfo] = {}
            name, dtype = ctypes.create_string_buffer(4096), ctypes.create_string_buffer(16)
            shape = (ctypes.c_longlong * 16)()
            begin, end = ctypes.c_longlong(), ctypes.c_longlong()
            for i in range(lib.mbl_count(handle)):
                ndim = lib.mbl_entry(handle, i, name, len(name), dtype, len(dtype), shape, len(shape), ctypes.byref(begin), ctypes.byref(end))
                if ndim < 0:
                    raise SafetensorsError(f"{path}: entry {i} of the header has a name or a shape too long to take")
                key = name.value.decode("utf-8")
                self.tensors[key] = TensorInfo(key, dtype.value.decode(), tuple(int(shape[k]) for k in range(ndim)), begin.value, end.value)
        finally:
            lib.mbl_close(handle)
        self._fh = open(path, "rb")
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if os.path.getsize(path) > 0 else None

    def names(self) -> List[str]:
        return list(self.tensors)

    def read(self, name: str) -> torch.Tensor:
        """The tensor as a CPU torch tensor in its stored dtype (a copy of the mapped bytes)."""
        info = self.tensors[name]
        dtype, _ = _DTYPES[info.dtype]
        raw = np.frombuffer(self._map, dtype=np.uint8, count=info.end - info.begin, offset=self.data_start + info.begin)
        flat = torch.from_numpy(raw.copy())
        return flat.view(dtype).reshape(info.shape)

    def close(self) -> None:
        if self._map is not None:
            self._map.close()
            self._map = None
        self._fh.close()


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]]) -> None:
    """Writes tensors in the order given; each is stored in its own dtype."""
    header: Dict[str, dict] = {}
    blobs: List[bytes] = []
    offset = 0
    for name, tensor in tensors:
        t = tensor.detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor `{name}`: dtype {t.dtype} cannot be stored")
        data = t.reshape(-1).view(torch.uint8).numpy().tobytes()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(data)]}
        blobs.append(data)
        offset += len(data)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * ((8 - len(text) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as fh:
        fh.write(struct.pack("<Q", len(text)))
        fh.write(text)
        for blob in blobs:
            fh.write(blob)
    os.replace(tmp, path)
