"""A plain, slow implementation of the Qwen3 dense decoder: whole sequences, no cache, one
function per part, torch on the CPU.  It shares no code with ``marin_b200``; it reads
``config.json`` with ``json`` and the weights with the ``safetensors`` library.

It rests on the reference's formulas (each function cites file:line in Kayleexx/marin); the
reference's own model code is Rust and cannot be compiled or imported here, so the anchor is
the reference's fixture ``tests/fixtures/tiny-qwen3`` with its ``reference.json`` (see
``tests/golden/``), which this file reproduces under the reference's own gate.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch


def read_config(model_dir: str) -> dict:
    """The keys the reference reads (crates/model/src/qwen3/config.rs:24-46) with its defaults
    (:87-96): kv heads default to heads, head_dim to hidden/heads, rope_theta may be nested."""
    with open(os.path.join(model_dir, "config.json")) as fh:
        raw = json.load(fh)
    heads = raw["num_attention_heads"]
    theta = raw.get("rope_theta")
    if theta is None:
        theta = raw["rope_parameters"]["rope_theta"]
    return {
        "layers": raw["num_hidden_layers"],
        "hidden": raw["hidden_size"],
        "heads": heads,
        "kv_heads": raw.get("num_key_value_heads") or heads,
        "head_dim": raw.get("head_dim") or raw["hidden_size"] // heads,
        "intermediate": raw["intermediate_size"],
        "vocab": raw["vocab_size"],
        "eps": float(raw["rms_norm_eps"]),
        "theta": float(theta),
        "tied": bool(raw.get("tie_word_embeddings", False)),
    }


def read_weights(model_dir: str, dtype=torch.float32) -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file

    return {k: v.to(dtype) for k, v in load_file(os.path.join(model_dir, "model.safetensors")).items()}


def as_bf16(x: torch.Tensor) -> torch.Tensor:
    """Rounds to bfloat16 and back: what a value loses when it is stored in 16 bits between two kernels."""
    return x.to(torch.bfloat16).to(torch.float32)


def same(x: torch.Tensor) -> torch.Tensor:
    return x


def embed(ids: Sequence[int], table: torch.Tensor) -> torch.Tensor:
    """hidden[t] = table[ids[t]], no scaling (crates/model/src/qwen3/model.rs:133-153)."""
    return table[torch.as_tensor(list(ids), dtype=torch.long)]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """ms = mean(x^2); y = x / sqrt(ms + eps) * w, weight multiplied directly
    (crates/tensor/src/norm.rs:16-22)."""
    mean_sq = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    return x * (1.0 / torch.sqrt(mean_sq + eps)) * weight


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """y[t][r] = sum_c w[r][c] x[t][c], no bias (crates/tensor/src/matrix.rs:128-131)."""
    return x @ w.t()


def rope(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """x: [T, heads, d].  f_i = theta^(-(2i/d)) in float32; angle = float(pos) * f_i; pair
    (a, b) = (x[i], x[i + d/2]) -> (a cos - b sin, b cos + a sin)
    (crates/tensor/src/ops.rs:52-95)."""
    d = x.shape[-1]
    half = d // 2
    i = torch.arange(half, dtype=torch.float32)
    freq = torch.pow(torch.tensor(theta, dtype=torch.float32), -(i * 2.0 / float(d)))
    angle = positions.to(torch.float32)[:, None] * freq[None, :]           # [T, half], float32
    cos, sin = torch.cos(angle).to(x.dtype)[:, None, :], torch.sin(angle).to(x.dtype)[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)


def softmax(scores: torch.Tensor) -> torch.Tensor:
    """m = max; e = exp(s - m); e / sum(e) (crates/tensor/src/ops.rs:23-33)."""
    e = torch.exp(scores - scores.max(dim=-1, keepdim=True).values)
    return e / e.sum(dim=-1, keepdim=True)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: Optional[int] = None, stored=same) -> torch.Tensor:
    """q: [T, H, d], k/v: [T, K, d].  Query head h reads kv head h // (H/K); scale 1/sqrt(d);
    token t sees positions 0..=t (crates/tensor/src/attention.rs:148-169).  ``window`` (not part
    of Qwen3) limits this to the last ``window`` positions.  ``stored`` is applied to the terms of
    the softmax before they meet the values (see ``forward``)."""
    T, H, d = q.shape
    K = k.shape[1]
    group = H // K
    scale = 1.0 / math.sqrt(d)
    out = torch.empty_like(q)
    for h in range(H):
        kh = h // group
        scores = (q[:, h, :] @ k[:, kh, :].t()) * scale                      # [T, T]
        idx = torch.arange(T)
        mask = idx[None, :] > idx[:, None]
        if window is not None:
            mask |= idx[None, :] < (idx[:, None] - window + 1)
        scores = scores.masked_fill(mask, float("-inf"))
        if stored is same:
            out[:, h, :] = softmax(scores) @ v[:, kh, :]
        else:
            # a 16-bit engine sums exp(s - m) in float32 but hands the terms to the value product in 16 bits
            e = torch.exp(scores - scores.max(dim=-1, keepdim=True).values)
            out[:, h, :] = (stored(e) @ v[:, kh, :]) / e.sum(dim=-1, keepdim=True)
    return out


def swiglu_mlp(x: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, stored=same) -> torch.Tensor:
    """down( g / (1 + exp(-g)) * u ) (crates/model/src/qwen3/mlp.rs:22-37, crates/tensor/src/silu.rs:18)."""
    g, u = linear(x, gate), linear(x, up)
    return linear(stored(g / (1.0 + torch.exp(-g)) * u), down)


def layer_forward(cfg: dict, w: Dict[str, torch.Tensor], n: int, hidden: torch.Tensor,
                  window: Optional[int] = None, kv_from=None, stored=same):
    """One pre-norm block (crates/model/src/qwen3/layer.rs:56-103): norm, q/k/v, per-head q/k norm
    before the rotation, causal attention, o_proj + residual, norm, SwiGLU + residual.  Returns the
    new hidden state and the (k, v) it attended over; ``kv_from`` makes it attend over given k, v.
    ``stored`` is applied to every value that a 16-bit engine keeps in 16 bits between two kernels (see ``forward``)."""
    p = f"model.layers.{n}."
    T = hidden.shape[0]
    H, K, d = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    pos = torch.arange(T)
    normed = stored(rms_norm(hidden, w[p + "input_layernorm.weight"], cfg["eps"]))
    q = stored(linear(normed, w[p + "self_attn.q_proj.weight"])).view(T, H, d)
    q = stored(rope(rms_norm(q, w[p + "self_attn.q_norm.weight"], cfg["eps"]), pos, cfg["theta"]))
    if kv_from is None:
        k = stored(linear(normed, w[p + "self_attn.k_proj.weight"])).view(T, K, d)
        v = stored(linear(normed, w[p + "self_attn.v_proj.weight"])).view(T, K, d)
        k = stored(rope(rms_norm(k, w[p + "self_attn.k_norm.weight"], cfg["eps"]), pos, cfg["theta"]))
    else:
        k, v = kv_from
    ctx = stored(attention(q, k, v, window, stored).reshape(T, H * d))
    hidden = hidden + linear(ctx, w[p + "self_attn.o_proj.weight"])
    normed = stored(rms_norm(hidden, w[p + "post_attention_layernorm.weight"], cfg["eps"]))
    hidden = hidden + swiglu_mlp(normed, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                                 w[p + "mlp.down_proj.weight"], stored)
    return hidden, (k, v)


def forward(cfg: dict, w: Dict[str, torch.Tensor], ids: Sequence[int], schedule: Optional[List[tuple]] = None,
            window: Optional[int] = None, return_hidden: bool = False, stored=same):
    """Logits [T, vocab] after every token of one whole sequence
    (crates/model/src/qwen3/model.rs:81-131; the reference keeps only the last row).
    ``schedule`` = [(layer, cache_of or None), ...] runs layers in another order (default 0..L-1).

    ``stored=as_bf16`` gives the model as an engine computes it that keeps activations in bfloat16 between
    kernels and everything else (sums, norms, softmax, the residual stream) in float32: the values the reference
    formulas produce are rounded where such an engine stores them (after each norm, the q/k/v projections, the
    per-head norm and rotation, the softmax terms, the attention output, the SwiGLU output).  Comparing a
    bfloat16 engine with this leaves only the differences of summation order and of where exactly a factor is
    applied, an order of magnitude less than the rounding itself."""
    hidden = embed(ids, w["model.embed_tokens.weight"])
    states = [hidden]
    schedule = schedule or [(n, None) for n in range(cfg["layers"])]
    kvs = []
    for layer, cache_of in schedule:
        hidden, kv = layer_forward(cfg, w, layer, hidden, window, kvs[cache_of] if cache_of is not None else None, stored)
        kvs.append(kv)
        states.append(hidden)
    normed = stored(rms_norm(hidden, w["model.norm.weight"], cfg["eps"]))
    head = w["model.embed_tokens.weight"] if cfg["tied"] else w["lm_head.weight"]
    logits = linear(normed, head)
    return (logits, states) if return_hidden else logits


def greedy(cfg: dict, w: Dict[str, torch.Tensor], prompt: Sequence[int], steps: int) -> List[int]:
    """Greedy continuation, recomputing the whole sequence at each step; lowest id wins ties
    (crates/sampler/src/lib.rs:40-48)."""
    ids = list(prompt)
    out = []
    for _ in range(steps):
        row = forward(cfg, w, ids)[-1]
        token = int(torch.argmax(row))  # torch.argmax returns the first maximal index
        out.append(token)
        ids.append(token)
    return out
