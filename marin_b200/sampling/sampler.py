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


def _total_order_key(values: np.ndarray) -> np.ndarray:
    """int32 keys that sort float32 values the way IEEE total order does (-0.0 below +0.0)."""
    bits = np.ascontiguousarray(values, dtype=np.float32).view(np.int32)
    return bits ^ ((bits >> 31) & np.int32(0x7FFFFFFF))


def best_index(values: np.ndarray) -> int:
    """Largest value, lowest index among equals (lib.rs:40-48)."""
    return int(np.argmax(_total_order_key(values)))


class Sampler:
    def __init__(self, params: SamplingParams):
        params.validate()
        self.params = params
        self.state = int(params.seed) & MASK64

    def next_unit(self) -> float:
        self.state = (self.state + 0x9E3779B97F4A7C15) & MASK64
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
        z ^= z >> 31
        return float(np.float32(z >> 40) / np.float32(16777216.0))

    def distribution(self, logits: np.ndarray, usable: Optional[int] = None) -> List[Tuple[int, float]]:
        logits = np.asarray(logits, dtype=np.float32).reshape(-1)
        usable = len(logits) if usable is None else usable
        if usable <= 0 or usable > len(logits):
            raise SamplerError(f"cannot sample from {usable} candidates out of {len(logits)} logits")
        cand = logits[:usable]
        if not np.all(np.isfinite(cand)):
            raise SamplerError("logits contain NaN or infinity")
        p = self.params
        if p.temperature == 0.0:
            return [(best_index(cand), 1.0)]
        key = _total_order_key(cand).astype(np.int64)
        order = np.argsort(-key, kind="stable")      # logit descending, id ascending among equals
        if p.top_k > 0:
            order = order[: p.top_k]
        ranked = cand[order]
        temperature = np.float32(p.temperature)
        weights = np.exp((ranked - ranked[0]) / temperature, dtype=np.float32)
        total = np.cumsum(weights, dtype=np.float32)[-1]
        probs = weights / total
        mass = np.cumsum(probs, dtype=np.float32)
        reached = np.nonzero(mass >= np.float32(p.top_p))[0]
        keep = int(reached[0]) + 1 if len(reached) else len(probs)
        kept = probs[:keep]
        kept_mass = np.cumsum(kept, dtype=np.float32)[-1]
        kept = kept / kept_mass
        return [(int(i), float(q)) for i, q in zip(order[:keep], kept)]

    def sample(self, logits: np.ndarray, usable: Optional[int] = None) -> int:
        dist = self.distribution(logits, usable)
        if self.params.temperature == 0.0:
            return dist[0][0]
        draw = np.float32(self.next_unit())
        cumulative = np.float32(0.0)
        for token, prob in dist:
            cumulative = np.float32(cumulative + np.float32(prob))
            if draw < cumulative:
                return token
        return dist[-1][0]
