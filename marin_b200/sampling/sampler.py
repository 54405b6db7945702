"""Token sampling with the reference's semantics (crates/sampler/src/lib.rs).

Order of operations (lib.rs:122-193): only the first ``usable`` logits are candidates; a NaN or
infinity is an error; temperature 0 picks the largest logit, the lowest id among equals;
otherwise tokens are ranked by (logit descending, id ascending), the best ``top_k`` are kept
(0 = all), weights ``exp((l - l_max) / temperature)`` are normalised, the shortest prefix whose
mass reaches ``top_p`` is kept (the crossing token included) and renormalised.  A draw
``u`` in [0, 1) from splitmix64 (top 24 bits, lib.rs:196-203) selects the first token whose
cumulative probability exceeds it, else the last (lib.rs:101-118).  Sums are float32 and
sequential.  The reference's two shortcuts (bounded top-k scan, the FAR cutoff) give the same
tokens as this plain algorithm by construction and are not repeated here.
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import numpy as np

MASK64 = (1 << 64) - 1


class SamplerError(ValueError):
    pass


@dataclass
class SamplingParams:
    """How one request is sampled and when it stops (names follow ``marin-run``'s flags,
    crates/cli/src/args.rs:352-389: --temp, --top-k, --top-p, --seed, --max-tokens)."""

    temperature: float = 0.7
    top_k: int = 0
    top_p: float = 0.9
    seed: int = 0
    max_tokens: int = 128
    stop_tokens: Sequence[int] = field(default_factory=tuple)
    #: ids at or above this are never sampled (model padding); None = the whole vocabulary
    usable_vocab: Optional[int] = None

    def validate(self) -> None:
        if not math.isfinite(self.temperature) or self.temperature < 0:
            raise SamplerError(f"temperature must be finite and >= 0, got {self.temperature}")
        if not (0.0 < self.top_p <= 1.0):
            raise SamplerError(f"top_p must be in (0, 1], got {self.top_p}")
        if self.top_k < 0:
            raise SamplerError(f"top_k must be >= 0, got {self.top_k}")
        if self.max_tokens < 0:
            raise SamplerError(f"max_tokens must be >= 0, got {self.max_tokens}")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0


def _host():
    from ..cache.pages import host_lib

    return host_lib()


def _row(values) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(values, dtype=np.float32).reshape(-1))


def best_index(values: np.ndarray) -> int:
    """Largest value under IEEE total order (-0.0 below +0.0), lowest index among equals (lib.rs:40-48)."""
    row = _row(values)
    return int(_host().mbp_best_index(row.ctypes.data, int(row.size)))


class Sampler:
    """One request's sampler: its parameters and its own splitmix64 stream.  The arithmetic is C++
    (``csrc/host/sampler.cpp``)."""

    def __init__(self, params: SamplingParams):
        params.validate()
        self.params = params
        self._state = ctypes.c_uint64(int(params.seed) & MASK64)
        self._lib = _host()

    @property
    def state(self) -> int:
        return int(self._state.value)

    def next_unit(self) -> float:
        return float(self._lib.mbp_next_unit(ctypes.byref(self._state)))

    @staticmethod
    def _raise(code: int, usable: int, size: int) -> None:
        if code == -1:
            raise SamplerError(f"cannot sample from {usable} candidates out of {size} logits")
        if code == -2:
            raise SamplerError("logits contain NaN or infinity")
        raise SamplerError(f"the sampler failed (code {code})")

    def distribution(self, logits: np.ndarray, usable: Optional[int] = None) -> List[Tuple[int, float]]:
        row = _row(logits)
        usable = int(row.size) if usable is None else int(usable)
        p = self.params
        cap = max(1, min(int(row.size), usable if usable > 0 else 1))
        ids, probs = np.zeros(cap, np.int32), np.zeros(cap, np.float32)
        kept = self._lib.mbp_distribution(row.ctypes.data, int(row.size), usable, float(p.temperature), int(p.top_k), float(p.top_p),
                                          ids.ctypes.data, probs.ctypes.data, cap)
        if kept < 0:
            self._raise(kept, usable, int(row.size))
        return [(int(i), float(q)) for i, q in zip(ids[:kept], probs[:kept])]

    def sample(self, logits: np.ndarray, usable: Optional[int] = None) -> int:
        row = _row(logits)
        usable = int(row.size) if usable is None else int(usable)
        p = self.params
        token = self._lib.mbp_sample(row.ctypes.data, int(row.size), usable, float(p.temperature), int(p.top_k), float(p.top_p),
                                     ctypes.byref(self._state))
        if token < 0:
            self._raise(token, usable, int(row.size))
        return int(token)
