"""Weights by tensor name from a model folder.

``model.safetensors`` or the shards of ``model.safetensors.index.json`` (``weight_map``) are
opened, compared with the list of tensors the model expects, and every problem found
is reported in ONE error: missing tensors, unexpected tensors, wrong shapes and wrong
dtypes (the reference collects them the same way, crates/model/src/qwen3/weights.rs:133-194;
sharding crates/loader/src/weights.rs:31-62,98-121).

Dtypes: bfloat16 stays bfloat16, a tensor stored in 32-bit stays 32-bit, integer tables
become int32.  Conversion to what a kernel wants happens when a part takes its tensor.
"""
from __future__ import annotations

import json
import os
import sys
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from ..parts.spec import TensorSpec
from .safetensors_io import SafetensorsError, SafetensorsFile

SINGLE = "model.safetensors"
INDEX = "model.safetensors.index.json"
MAX_LISTED = 12

_FLOAT_OK = {"BF16", "F32"}
_INT_OK = {"I8", "U8", "I16", "I32", "I64"}


class WeightError(ValueError):
    """The checkpoint does not hold what the model expects; the message lists everything wrong."""

    def __init__(self, problems: Sequence[str], where: str):
        self.problems = list(problems)
        shown = self.problems[:MAX_LISTED]
        more = len(self.problems) - len(shown)
        text = f"{where}: {len(self.problems)} problem(s) with the weights:\n  " + "\n  ".join(shown)
        if more > 0:
            text += f"\n  ... and {more} more"
        super().__init__(text)


class Checkpoint:
    """All tensors of a model folder, whichever file holds them."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        self.files: List[SafetensorsFile] = []
        self.owner: Dict[str, SafetensorsFile] = {}
        single = os.path.join(model_dir, SINGLE)
        index = os.path.join(model_dir, INDEX)
        if os.path.exists(single):
            paths = [single]
        elif os.path.exists(index):
            with open(index, "r", encoding="utf-8") as fh:
                weight_map = json.load(fh).get("weight_map")
            if not isinstance(weight_map, dict) or not weight_map:
                raise SafetensorsError(f"{index}: no `weight_map`")
            paths = [os.path.join(model_dir, f) for f in sorted(set(weight_map.values()))]
            missing = [p for p in paths if not os.path.exists(p)]
            if missing:
                raise SafetensorsError(f"{model_dir}: shard(s) named by the index are missing: {missing}")
        else:
            raise SafetensorsError(f"{model_dir}: neither {SINGLE} nor {INDEX} found")
        for path in paths:
            f = SafetensorsFile(path)
            self.files.append(f)
            for name in f.names():
                if name in self.owner:
                    raise SafetensorsError(f"tensor `{name}` is in both {self.owner[name].path} and {path}")
                self.owner[name] = f

    def names(self) -> List[str]:
        return list(self.owner)

    def info(self, name: str):
        return self.owner[name].tensors[name]

    def read(self, name: str) -> torch.Tensor:
        return self.owner[name].read(name)

    def close(self) -> None:
        for f in self.files:
            f.close()


def check(ckpt: Checkpoint, expected: Iterable[TensorSpec], ignorable: Sequence[str] = (),
          extras: Optional[List[str]] = None) -> List[str]:
    """Every mismatch between the checkpoint and the expected tensors, as readable lines.  Tensors of the checkpoint
    that the model does not know are problems too, unless ``extras`` is a list: their names then go there."""
    problems: List[str] = []
    wanted = {}
    for spec in expected:
        wanted[spec.name] = spec
    have = set(ckpt.names())
    for name, spec in wanted.items():
        if name not in have:
            problems.append(f"missing tensor `{name}` {list(spec.shape)}")
            continue
        info = ckpt.info(name)
        if tuple(info.shape) != tuple(spec.shape):
            problems.append(f"tensor `{name}` has shape {list(info.shape)} but config.json implies {list(spec.shape)}")
        ok = _INT_OK if spec.role == "int_table" else _FLOAT_OK
        if info.dtype not in ok:
            problems.append(f"tensor `{name}` is {info.dtype} but expected one of {sorted(ok)}")
    for name in sorted(have - set(wanted) - set(ignorable)):
        if extras is not None:
            extras.append(name)
        else:
            problems.append(f"unexpected tensor `{name}` {list(ckpt.info(name).shape)}")
    return problems


def load_tensors(model_dir: str, expected: Sequence[TensorSpec], ignorable: Sequence[str] = (), extra_tensors: str = "error",
                 ignored: Optional[List[str]] = None) -> Dict[str, torch.Tensor]:
    """name → CPU tensor in its stored dtype (ints as int32), after the checkpoint passed ``check``.

    ``extra_tensors`` says what tensors the model does not know are: ``"error"`` (the default) lists them in the one
    ``WeightError`` with everything else that is wrong; ``"warn"`` leaves them unread, appends their names to
    ``ignored`` if a list is given and says so once on stderr (the reference reads only what it expects and ignores
    the rest: crates/model/src/qwen3/weight_bytes.rs:9-10)."""
    if extra_tensors not in ("error", "warn"):
        raise ValueError(f"extra_tensors must be 'error' or 'warn', got {extra_tensors!r}")
    ckpt = Checkpoint(model_dir)
    try:
        extras: Optional[List[str]] = [] if extra_tensors == "warn" else None
        problems = check(ckpt, expected, ignorable, extras)
        if problems:
            raise WeightError(problems, model_dir)
        if extras:
            shown = ", ".join(f"`{n}`" for n in extras[:MAX_LISTED]) + (f" and {len(extras) - MAX_LISTED} more" if len(extras) > MAX_LISTED else "")
            print(f"[marin_b200] {model_dir}: {len(extras)} tensor(s) the model does not know were left unread: {shown}", file=sys.stderr)
            if ignored is not None:
                ignored.extend(extras)
        out: Dict[str, torch.Tensor] = {}
        for spec in expected:
            t = ckpt.read(spec.name)
            if spec.role == "int_table":
                t = t.to(torch.int32)
            out[spec.name] = t
        return out
    finally:
        ckpt.close()
