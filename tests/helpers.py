"""Shared by the tests: the tiny configurations, model folders in temporary places, and ways of
cutting requests into steps."""
from __future__ import annotations

import json
import os
import random
from typing import Dict, List, Sequence, Tuple

import torch

# Tiny configurations that differ in every size and option the architecture has.
TINY_A = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 2, "hidden_size": 64,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 128, "vocab_size": 256,
    "rope_theta": 10000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 128,
    "hidden_act": "silu",
}
TINY_B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 3, "hidden_size": 96,
    "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 32, "intermediate_size": 320, "vocab_size": 384,
    "rope_parameters": {"rope_theta": 1000000.0, "rope_type": "default"}, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False, "max_position_embeddings": 256,
}
# Sizes that are no power of two anywhere: 6 heads in 3 groups of head size 48, odd vocabulary.
TINY_C = {
    "model_type": "qwen3", "num_hidden_layers": 1, "hidden_size": 72, "num_attention_heads": 6,
    "num_key_value_heads": 3, "head_dim": 48, "intermediate_size": 136, "vocab_size": 333, "rope_theta": 500000.0,
    "rms_norm_eps": 3e-6, "tie_word_embeddings": False, "max_position_embeddings": 192,
}
# Heads of 128 and a width that lets the matrix products cut K: the layout the tensor-core attention kernels, the TMA
# decode kernel and the fused epilogues (heads finished by the q|k|v product, norms riding on products) are made for.
TINY_D = {
    "model_type": "qwen3", "num_hidden_layers": 2, "hidden_size": 512, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 640, "vocab_size": 500, "rope_theta": 1000000.0,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 160,
}
PAGE = {"A": 4, "B": 8, "C": 16, "D": 16}
# Standard deviation of the random matrices: about 1 / sqrt(width), so that logits keep a standard deviation near 1
# (the bfloat16 tolerances are absolute and stated for such logits).
MATRIX_STD = {"A": 0.1, "B": 0.1, "C": 0.1, "D": 0.05}
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D}


def make_model_dir(path: str, raw: dict, seed: int, dtype=torch.float32, matrix_std: float = 0.02) -> str:
    """config.json + model.safetensors with random weights, through the engine's random-weights mode.
    (The plain implementation reads the folder back with its own code.)"""
    from marin_b200.config import Qwen3Config
    from marin_b200.weights import write_random_model

    cfg = Qwen3Config.from_dict(raw)
    write_random_model(path, cfg, seed, dtype, matrix_std=matrix_std)
    # keep the raw keys (nested rope_parameters and the like) so that parsing them is exercised
    with open(os.path.join(path, "config.json"), "w") as fh:
        json.dump(raw, fh)
    return path


def random_prompt(rng: random.Random, vocab: int, n: int) -> List[int]:
    return [rng.randrange(vocab) for _ in range(n)]


def portions(total: int, sizes: Sequence[int]) -> List[int]:
    """Cuts ``total`` tokens into portions whose sizes cycle through ``sizes``."""
    out, i = [], 0
    while total > 0:
        n = min(total, sizes[i % len(sizes)])
        out.append(n)
        total -= n
        i += 1
    return out


def run_whole(runner, req_id, tokens) -> torch.Tensor:
    """One request alone, whole, logits at every place."""
    from marin_b200.engine import StepEntry

    runner.begin(req_id)
    logits = runner.step([StepEntry(req_id, list(tokens), list(range(len(tokens))))]).clone()
    runner.end(req_id)
    return logits


def run_portions(runner, req_id, tokens, sizes: Sequence[int]) -> torch.Tensor:
    """One request alone, in the given portions, logits at every place."""
    from marin_b200.engine import StepEntry

    runner.begin(req_id)
    rows, at = [], 0
    for n in sizes:
        rows.append(runner.step([StepEntry(req_id, list(tokens[at:at + n]), list(range(n)))]).clone())
        at += n
    assert at == len(tokens)
    runner.end(req_id)
    return torch.cat(rows, dim=0)


def mixed_schedule(rng: random.Random, lengths: Dict[str, int], max_live: int = 4, decode_tail: int = 6,
                   sizes: Sequence[int] = (7, 2, 13, 3, 2, 5)) -> List[Tuple[List[Tuple[str, int]], List[str]]]:
    """Steps [(entries [(id, n)], ends [id])]: up to ``max_live`` requests live at once; each is fed
    in portions of changing size and its last ``decode_tail`` tokens one by one, so that portions of
    some requests run beside single tokens of others; a request ends as soon as it is fed, which
    gives its pages back for the next one to use."""
    waiting = list(lengths)
    live: Dict[str, List[int]] = {}
    steps = []
    k = 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid = waiting.pop(0)
            n = lengths[rid]
            tail = min(decode_tail, max(0, n - 1))
            plan = portions(n - tail, sizes[k % len(sizes):] + sizes[:k % len(sizes)]) + [1] * tail
            live[rid] = plan
            k += 1
        entries, ends = [], []
        for rid in list(live):
            if rng.random() < 0.2 and len(live) > 1:
                continue                       # a request may be left out of a step and go on later
            n = live[rid].pop(0)
            entries.append((rid, n))
            if not live[rid]:
                ends.append(rid)
                del live[rid]
        if entries:
            steps.append((entries, ends))
    return steps


def run_mixed(runner, tokens: Dict[str, List[int]], steps) -> Dict[str, torch.Tensor]:
    """Runs a mixed schedule asking for logits everywhere; returns per request logits [len, vocab]."""
    from marin_b200.engine import StepEntry

    fed = {rid: 0 for rid in tokens}
    rows: Dict[str, List[torch.Tensor]] = {rid: [] for rid in tokens}
    begun = set()
    for entries, ends in steps:
        batch = []
        for rid, n in entries:
            if rid not in begun:
                runner.begin(rid)
                begun.add(rid)
            batch.append(StepEntry(rid, tokens[rid][fed[rid]:fed[rid] + n], list(range(n))))
        logits = runner.step(batch).clone()
        at = 0
        for rid, n in entries:
            rows[rid].append(logits[at:at + n])
            at += n
            fed[rid] += n
        for rid in ends:
            runner.end(rid)
    return {rid: torch.cat(r, dim=0) for rid, r in rows.items()}
