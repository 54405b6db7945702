"""Plain torch versions of every kernel, with the kernels' own signatures.

Two uses, both in tests only: (1) each CUDA kernel is compared with its function here, alone,
at sizes other than the engine's; (2) ``patch_ops`` puts these functions in place of the CUDA
kernels so that the host logic of the engine (batching, block tables, commits) can be
exercised on a machine without a GPU.  The product never imports this file.
"""
from __future__ import annotations

import math
from contextlib import contextmanager

import torch


def embed(ids, table, out):
    out.copy_(table[ids.long()].float())


def rmsnorm(x, weight, eps, out, unit_offset=False):
    xf = x.float()
    ms = (xf * xf).sum(-1, keepdim=True) / xf.shape[-1]
    w = weight.float() + 1.0 if unit_offset else weight.float()
    out.copy_((xf * (1.0 / torch.sqrt(ms + eps)) * w).to(out.dtype))


def gemm(x, w, out, accumulate=False, then_norm=None):
    y = x.float() @ w.float().t()
    if accumulate:
        out.add_(y.to(out.dtype))
    else:
        out.copy_(y.to(out.dtype))


def gemm_qkv_heads(*args, **kwargs):
    return False


def qk_norm_rope_write(qkv, q_out, q_weight, k_weight, eps, positions, inv_freq, rotary_dim, interleaved,
                       slot_mapping, k_cache, v_cache, H, K, d, write_kv=True):
    T = qkv.shape[0]
    heads_total = H + 2 * K if write_kv else H
    x = qkv.float().view(T, heads_total, d).clone()

    def norm(part, w):
        if w is None:
            return part
        ms = (part * part).sum(-1, keepdim=True) / d
        return part * (1.0 / torch.sqrt(ms + eps)) * w.float()

    def rotate(part):
        if inv_freq is None:
            return part
        half = rotary_dim // 2
        ang = positions.float()[:, None] * inv_freq.float()[None, :]
        cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        part = part.clone()
        if interleaved:
            a, b = part[..., 0:rotary_dim:2].clone(), part[..., 1:rotary_dim:2].clone()
            part[..., 0:rotary_dim:2] = a * cos - b * sin
            part[..., 1:rotary_dim:2] = b * cos + a * sin
        else:
            a, b = part[..., :half].clone(), part[..., half:rotary_dim].clone()
            part[..., :half] = a * cos - b * sin
            part[..., half:rotary_dim] = b * cos + a * sin
        return part

    q = rotate(norm(x[:, :H], q_weight))
    q_out.copy_(q.reshape(T, H * d).to(q_out.dtype))
    if not write_kv:
        return
    k = rotate(norm(x[:, H:H + K], k_weight))
    v = x[:, H + K:]
    page_size = k_cache.shape[2]
    slots = slot_mapping.long()
    ok = slots >= 0
    page, off = slots[ok] // page_size, slots[ok] % page_size
    k_cache[page, :, off, :] = k[ok].to(k_cache.dtype)
    v_cache[page, :, off, :] = v[ok].to(v_cache.dtype)


def attention(q, k_cache, v_cache, out, ctx, block_table, H, K, d, scale, window=0, plan=None):
    T = q.shape[0]
    page_size = k_cache.shape[2]
    group = H // K
    qf = q.float().view(T, H, d)
    res = torch.zeros(T, H, d, dtype=torch.float32, device=q.device)
    positions = ctx.positions.tolist()
    reqs = ctx.req_index.tolist()
    head_kv = torch.arange(H, device=q.device) // group
    for t in range(T):
        pos, r = positions[t], reqs[t]
        lo = max(0, pos - window + 1) if window > 0 else 0
        keys = torch.arange(lo, pos + 1, device=q.device)
        pages = block_table[r].long()[keys // page_size]
        kk = k_cache[pages, :, keys % page_size, :].float()[:, head_kv, :]   # [n, H, d]
        vv = v_cache[pages, :, keys % page_size, :].float()[:, head_kv, :]
        s = torch.einsum("nhd,hd->hn", kk, qf[t]) * scale
        p = torch.softmax(s, dim=-1)
        res[t] = torch.einsum("hn,nhd->hd", p, vv)
    out.copy_(res.view(T, H * d).to(out.dtype))


def swiglu(gate_up, out, interleaved=False):
    T, I = out.shape
    if interleaved:
        blocks = gate_up.float().view(T, I // 16, 2, 16)
        g, u = blocks[:, :, 0, :].reshape(T, I), blocks[:, :, 1, :].reshape(T, I)
    else:
        g, u = gate_up[:, :I].float(), gate_up[:, I:].float()
    out.copy_((g / (1.0 + torch.exp(-g)) * u).to(out.dtype))


def interleave_gate_up(gate, up):
    I, h = gate.shape
    return torch.stack([gate.view(I // 16, 16, h), up.view(I // 16, 16, h)], dim=1).reshape(2 * I, h)


def can_fuse_swiglu(dtype, hidden, intermediate):
    return dtype == torch.bfloat16 and intermediate % 16 == 0 and hidden % 8 == 0


def gemm_swiglu(x, w_interleaved, out, workspace=None):
    y = x.float() @ w_interleaved.float().t()
    swiglu(y, out, interleaved=True)


def gather_rows(src, rows, out):
    out.copy_(src[rows.long()])


def add_into(y, x):
    y.add_(x.float().view_as(y))


def argmax(logits, usable, out):
    out.copy_(torch.argmax(logits[:, :usable], dim=-1).to(torch.int32))


def sample(logits, usable, temperature, top_k, top_p, uniform, out):
    """The host sampler's kept set, walked in id order."""
    import numpy as np

    from marin_b200.sampling import Sampler, SamplingParams
    for r in range(logits.shape[0]):
        t, k, p = float(temperature[r]), int(top_k[r]), float(top_p[r])
        dist = Sampler(SamplingParams(temperature=t, top_k=k, top_p=p)).distribution(logits[r].float().cpu().numpy(), int(usable[r]))
        dist.sort()
        target, run, pick = float(uniform[r]), 0.0, dist[-1][0]
        for token, prob in dist:
            if run <= target < run + prob:
                pick = token
                break
            run += prob
        out[r] = pick


NAMES = ["sample", "embed", "rmsnorm", "gemm", "qk_norm_rope_write", "attention", "swiglu", "gather_rows", "add_into", "argmax",
         "interleave_gate_up", "can_fuse_swiglu", "gemm_swiglu", "gemm_qkv_heads"]


@contextmanager
def patch_ops():
    """Swaps the CUDA kernels for the functions above (host-logic tests on a machine without a GPU)."""
    from marin_b200.kernels import ops

    saved = {n: getattr(ops, n, None) for n in NAMES}
    try:
        for n in NAMES:
            setattr(ops, n, globals()[n])
        yield
    finally:
        for n, f in saved.items():
            if f is None:
                delattr(ops, n)
            else:
                setattr(ops, n, f)
