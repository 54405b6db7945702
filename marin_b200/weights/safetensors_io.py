"""Reading and writing the safetensors container.

Layout (the same the reference parses, crates/loader/src/safetensors.rs:54-106):
8 bytes little-endian header length, a JSON header mapping tensor name to
``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to the end of
the header), then the raw little-endian tensor bytes.  The file is memory-mapped;
tensors are views until they are copied to the device.
"""
from __future__ import annotations

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
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to hold a safetensors header (partial download?)")
        self._fh = open(path, "rb")
        (header_len,) = struct.unpack("<Q", self._fh.read(8))
        if header_len > MAX_HEADER_BYTES or 8 + header_len > size:
            raise SafetensorsError(f"{path}: header of {header_len} bytes does not fit the file (partial download?)")
        try:
            header = json.loads(self._fh.read(header_len).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as err:
            raise SafetensorsError(f"{path}: header is not valid JSON: {err}") from err
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        self.data_start = 8 + header_len
        data_bytes = size - self.data_start
        self.tensors: Dict[str, TensorInfo] = {}
        for name, entry in header.items():
            if name == "__metadata__":
                continue
            try:
                dtype = entry["dtype"]
                shape = tuple(int(s) for s in entry["shape"])
                begin, end = (int(v) for v in entry["data_offsets"])
            except (KeyError, TypeError, ValueError) as err:
                raise SafetensorsError(f"{path}: malformed entry for tensor `{name}`") from err
            if dtype not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor `{name}` has unsupported dtype {dtype}")
            count = 1
            for s in shape:
                if s < 0:
                    raise SafetensorsError(f"{path}: tensor `{name}` has a negative size")
                count *= s
            if begin < 0 or end < begin or end - begin != count * _DTYPES[dtype][1]:
                raise SafetensorsError(f"{path}: tensor `{name}`: offsets {begin}..{end} do not match shape {shape} {dtype}")
            if end > data_bytes:
                raise SafetensorsError(f"{path}: tensor `{name}` ends at byte {end} but the file holds {data_bytes} (partial download?)")
            self.tensors[name] = TensorInfo(name, dtype, shape, begin, end)
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

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
