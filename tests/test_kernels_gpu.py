"""Each CUDA kernel alone against its plain torch twin (tests/kernel_refs.py), at sizes other than
the engine's: widths and vocabularies that are no power of two, head sizes in steps of 16, odd
head counts and groups, scrambled block tables, windows."""
import math
import random
from types import SimpleNamespace

import pytest
import torch

import kernel_refs as ref

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(rtol=2e-5, atol=2e-6) if dtype == torch.float32 else dict(rtol=1.6e-2, atol=1e-3)


@pytest.fixture(scope="module")
def ops():
    from marin_b200.kernels import ops as o
    return o


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("vocab,h,tokens", [(333, 72, 5), (1000, 2560, 37), (17, 8, 1)])
def test_embed(ops, dtype, vocab, h, tokens):
    g = torch.Generator(device=DEV).manual_seed(1)
    table = torch.randn(vocab, h, device=DEV, generator=g).to(dtype)
    ids = torch.randint(0, vocab, (tokens,), device=DEV, generator=g, dtype=torch.int32)
    ids[0] = vocab - 1
    out, want = torch.empty(tokens, h, device=DEV), torch.empty(tokens, h, device=DEV)
    ops.embed(ids, table, out)
    ref.embed(ids, table, want)
    assert torch.equal(out, want)


@pytest.mark.parametrize("out_dtype", DTYPES)
@pytest.mark.parametrize("rows,n,eps,unit", [(3, 72, 1e-5, False), (17, 2560, 1e-6, False), (300, 4096, 1e-6, True), (33, 5120, 1e-6, False), (2, 8192, 1e-6, False), (9, 512, 1e-5, False), (4, 4092, 1e-6, False), (1, 5120, 1e-6, True), (5, 1, 1e-3, False), (2, 1031, 1e-6, False)])
def test_rmsnorm(ops, out_dtype, rows, n, eps, unit):
    g = torch.Generator(device=DEV).manual_seed(2)
    x = torch.randn(rows, n, device=DEV, generator=g) * 3.0
    w = 1.0 + 0.2 * torch.randn(n, device=DEV, generator=g)
    out, want = torch.empty(rows, n, device=DEV, dtype=out_dtype), torch.empty(rows, n, device=DEV, dtype=out_dtype)
    ops.rmsnorm(x, w, eps, out, unit)
    ref.rmsnorm(x.double(), w.double(), eps, want, unit)
    torch.testing.assert_close(out.float(), want.float(), **tol(out_dtype))


GEMM_SHAPES = [(1, 72, 72), (5, 333, 136), (64, 256, 64), (65, 130, 200), (16, 1000, 2560), (130, 96, 1031), (8, 384, 96)]


@pytest.mark.parametrize("combo", ["f32", "bf16", "bf16_f32out"])
@pytest.mark.parametrize("T,N,K", GEMM_SHAPES)
def test_gemm(ops, combo, T, N, K):
    g = torch.Generator(device=DEV).manual_seed(3)
    in_dtype = torch.float32 if combo == "f32" else torch.bfloat16
    out_dtype = torch.bfloat16 if combo == "bf16" else torch.float32
    x = torch.randn(T, K, device=DEV, generator=g).to(in_dtype)
    w = (torch.randn(N, K, device=DEV, generator=g) / math.sqrt(K)).to(in_dtype)
    out = torch.empty(T, N, device=DEV, dtype=out_dtype)
    ops.gemm(x, w, out)
    want = (x.double() @ w.double().t())
    torch.testing.assert_close(out.double(), want, **(dict(rtol=1e-5, atol=1e-5) if out_dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)))
    if out_dtype == torch.float32:
        base = torch.randn(T, N, device=DEV, generator=g)
        acc = base.clone()
        ops.gemm(x, w, acc, accumulate=True)
        torch.testing.assert_close(acc.double(), base.double() + want, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("T", [24, 32, 16, 64])
def test_gemm_of_a_few_tokens_many_times_back_to_back_gives_the_same_bits(ops, T):
    """The small-batch product has two MMA issuers that share one ring of stages; launched back to back (each launch a
    programmatic dependent of the one before, as in a decode step) its K slices start at different moments every time.
    Three hundred launches at a layer's real sizes must give one and the same result, the right one."""
    g = torch.Generator(device=DEV).manual_seed(40 + T)
    N, K = 2560, 9728
    x = torch.randn(T, K, device=DEV, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    outs = torch.empty(300, T, N, device=DEV, dtype=torch.float32)
    for i in range(300):
        ops.gemm(x, w, outs[i])
    ops.check_device_errors()
    want = x.double() @ w.double().t()
    torch.testing.assert_close(outs[0].double(), want, rtol=1e-5, atol=1e-5)
    same = (outs == outs[0]).flatten(1).all(dim=1)
    assert bool(same.all()), f"launch {int(torch.nonzero(~same)[0])} of 300 gave other bits than the first"


@pytest.mark.parametrize("T,N,K", [(1000, 2560, 512), (2048, 2560, 4096), (777, 3000, 320), (1500, 1981, 256), (1031, 4100, 192)])
def test_gemm_of_many_tokens_adds_into_float32(ops, T, N, K):
    """``out += x w^T`` in the persistent kernel (by TMA reduction where the rows of ``out`` can be a tensor map's: N a
    multiple of 4; by read and write otherwise), with token counts and widths that leave partial tiles, against
    float64; twice, so that a second launch adds to what the first left."""
    g = torch.Generator(device=DEV).manual_seed(50)
    assert ops.many_tokens(T, N)
    x = torch.randn(T, K, device=DEV, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    base = torch.randn(T, N, device=DEV, generator=g)
    guard = torch.full((T + 2, N), 7.0, device=DEV)             # rows around the matrix: nothing may be written there
    out = guard[1:T + 1]
    out.copy_(base)
    product = x.double() @ w.double().t()
    ops.gemm(x, w, out, accumulate=True)
    torch.testing.assert_close(out.double(), base.double() + product, rtol=1e-5, atol=2e-5)
    ops.gemm(x, w, out, accumulate=True)
    torch.testing.assert_close(out.double(), base.double() + 2 * product, rtol=1e-5, atol=4e-5)
    assert bool((guard[0] == 7.0).all()) and bool((guard[T + 1] == 7.0).all())
    ops.check_device_errors()


def test_gemm_rows_do_not_depend_on_the_batch(ops):
    """A row's result is the same alone and among 200 other rows (float32 path: bit for bit)."""
    g = torch.Generator(device=DEV).manual_seed(4)
    x = torch.randn(201, 320, device=DEV, generator=g)
    w = torch.randn(96, 320, device=DEV, generator=g)
    full, one = torch.empty(201, 96, device=DEV), torch.empty(1, 96, device=DEV)
    ops.gemm(x, w, full)
    ops.gemm(x[137:138].contiguous(), w, one)
    assert torch.equal(full[137:138], one)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,K,d,rot,inter,norm,page", [(4, 2, 16, 16, False, True, 4), (6, 3, 48, 48, False, True, 16), (8, 2, 128, 128, False, True, 16),
                                                       (5, 5, 32, 16, True, False, 8), (3, 1, 80, 80, False, True, 2), (2, 2, 256, 256, False, True, 32),
                                                       (7, 1, 64, 64, False, True, 16), (40, 8, 128, 128, False, False, 16), (4, 4, 128, 64, False, True, 16)])
def test_qk_norm_rope_write(ops, dtype, H, K, d, rot, inter, norm, page):
    g = torch.Generator(device=DEV).manual_seed(5)
    T, pages = (23, 12) if d != 48 else (300, 24)        # many tokens take the one-CTA-per-token path
    qkv = torch.randn(T, (H + 2 * K) * d, device=DEV, generator=g).to(dtype)
    qw = (1 + 0.1 * torch.randn(d, device=DEV, generator=g)) if norm else None
    kw = (1 + 0.1 * torch.randn(d, device=DEV, generator=g)) if norm else None
    positions = torch.randint(0, 4000, (T,), device=DEV, generator=g, dtype=torch.int32)
    inv_freq = torch.pow(torch.tensor(1e6), -(torch.arange(rot // 2, dtype=torch.float32) * 2.0 / rot)).to(DEV)
    slots = torch.randperm(pages * page, device=DEV, generator=g)[:T].to(torch.int32)
    slots[3] = -1      # a padded token writes nothing
    caches = [torch.zeros(pages, K, page, d, device=DEV, dtype=dtype) for _ in range(4)]
    q1, q2 = torch.empty(T, H * d, device=DEV, dtype=dtype), torch.empty(T, H * d, device=DEV, dtype=dtype)
    ops.qk_norm_rope_write(qkv, q1, qw, kw, 1e-6, positions, inv_freq, rot, inter, slots, caches[0], caches[1], H, K, d, True)
    ref.qk_norm_rope_write(qkv, q2, qw, kw, 1e-6, positions, inv_freq, rot, inter, slots, caches[2], caches[3], H, K, d, True)
    t = dict(rtol=1e-4, atol=2e-4) if dtype == torch.float32 else dict(rtol=1.6e-2, atol=2e-2)
    torch.testing.assert_close(q1.float(), q2.float(), **t)
    torch.testing.assert_close(caches[0].float(), caches[2].float(), **t)
    assert torch.equal(caches[1], caches[3])       # values are copied unchanged
    # queries only (a layer that reads another layer's cache)
    q_only = qkv[:, : H * d].contiguous()
    q3 = torch.empty_like(q1)
    before = caches[0].clone()
    ops.qk_norm_rope_write(q_only, q3, qw, kw, 1e-6, positions, inv_freq, rot, inter, slots, caches[0], caches[1], H, K, d, False)
    assert torch.equal(q3, q1) and torch.equal(caches[0], before)


def paged_case(gen, dtype, lens_new, H, K, d, page, pages, scale_far=None):
    """Requests [(cached, new)] with scrambled block tables and a filled cache."""
    R = len(lens_new)
    maxb = max(-(-(c + n) // page) for c, n in lens_new) + 1
    perm = torch.randperm(pages, generator=gen, device=DEV).tolist()
    table = torch.zeros(R, maxb, dtype=torch.int32, device=DEV)
    at = 0
    positions, req_index = [], []
    for r, (c, n) in enumerate(lens_new):
        nb = -(-(c + n) // page)
        table[r, :nb] = torch.tensor(perm[at:at + nb], dtype=torch.int32)
        at += nb
        positions += list(range(c, c + n))
        req_index += [r] * n
    assert at <= pages
    T = len(positions)
    k_cache = torch.randn(pages, K, page, d, device=DEV, generator=gen).to(dtype)
    v_cache = torch.randn(pages, K, page, d, device=DEV, generator=gen).to(dtype)
    q = torch.randn(T, H * d, device=DEV, generator=gen).to(dtype)
    ctx = SimpleNamespace(
        positions=torch.tensor(positions, dtype=torch.int32, device=DEV),
        req_index=torch.tensor(req_index, dtype=torch.int32, device=DEV),
        cu_tokens=torch.tensor([0] + list(torch.tensor([n for _, n in lens_new]).cumsum(0)), dtype=torch.int32, device=DEV),
        seq_lens=torch.tensor([c + n for c, n in lens_new], dtype=torch.int32, device=DEV),
        num_tokens=T, num_requests=R, num_decode=sum(1 for _, n in lens_new if n == 1),
        max_query_len=max(n for _, n in lens_new), max_seq_len=max(c + n for c, n in lens_new),
    )
    return q, k_cache, v_cache, table, ctx


ATT_LAYOUTS = [(4, 2, 16, 4), (8, 2, 32, 8), (6, 3, 48, 16), (32, 8, 128, 16), (5, 1, 64, 16), (3, 3, 80, 32), (2, 1, 256, 64)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,K,d,page", ATT_LAYOUTS)
@pytest.mark.parametrize("window", [0, 37])
def test_attention_mixed_batch(ops, dtype, H, K, d, page, window):
    g = torch.Generator(device=DEV).manual_seed(6)
    # decodes first (as the step function orders them), then prompt portions, some from position 0
    lens_new = [(130, 1), (63, 1), (0, 1), (255, 1), (0, 70), (129, 65), (17, 2), (64, 128)]
    pages = sum(-(-(c + n) // page) for c, n in lens_new) + 3
    q, kc, vc, table, ctx = paged_case(g, dtype, lens_new, H, K, d, page, pages)
    out, want = torch.empty_like(q), torch.empty_like(q)
    scale = 1.0 / math.sqrt(d)
    ops.attention(q, kc, vc, out, ctx, table, H, K, d, scale, window)
    ref.attention(q, kc, vc, want, ctx, table, H, K, d, scale, window)
    t = dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(out.float(), want.float(), **t)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("context", [1, 15, 16, 17, 127, 128, 129, 255, 256, 257, 1023, 1025, 2049])
def test_attention_decode_at_page_and_chunk_edges(ops, dtype, context):
    g = torch.Generator(device=DEV).manual_seed(7)
    H, K, d, page = 8, 2, 64, 16
    lens_new = [(context - 1, 1), (max(0, context - 3), 1)]
    pages = sum(-(-(c + n) // page) for c, n in lens_new) + 2
    q, kc, vc, table, ctx = paged_case(g, dtype, lens_new, H, K, d, page, pages)
    out, want = torch.empty_like(q), torch.empty_like(q)
    ops.attention(q, kc, vc, out, ctx, table, H, K, d, 0.125, 0)
    ref.attention(q, kc, vc, want, ctx, table, H, K, d, 0.125, 0)
    t = dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(out.float(), want.float(), **t)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("far_key", [0, 3, 15, 16, 511, 640, 700])
def test_attention_finds_one_far_key_among_hundreds(ops, dtype, far_key):
    """Random inputs spread attention thinly, so a skipped key would hardly show.  Here one key far
    back matches the query exactly and strongly: the output must be that key's value."""
    g = torch.Generator(device=DEV).manual_seed(8)
    H, K, d, page = 4, 2, 32, 16
    lens_new = [(700, 1), (690, 11)]
    pages = sum(-(-(c + n) // page) for c, n in lens_new) + 1
    q, kc, vc, table, ctx = paged_case(g, dtype, lens_new, H, K, d, page, pages)
    kc.mul_(0.05)
    # token 0 (request 0) and the last token of request 1: every head's query is twice the far key
    # of its kv head, whose norm is 6: that score is 72, all others stay near 0
    for t_idx, r in ((0, 0), (11, 1)):
        pg = int(table[r, far_key // page])
        for kh in range(K):
            key = torch.randn(d, device=DEV, generator=g)
            kc[pg, kh, far_key % page] = (key / key.norm() * 6).to(dtype)
        for h in range(H):
            q.view(-1, H, d)[t_idx, h] = (kc[pg, h // (H // K), far_key % page].float() * 2).to(dtype)
    out, want = torch.empty_like(q), torch.empty_like(q)
    ops.attention(q, kc, vc, out, ctx, table, H, K, d, 1.0, 0)
    ref.attention(q, kc, vc, want, ctx, table, H, K, d, 1.0, 0)
    t = dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(out.float(), want.float(), **t)
    for t_idx, r in ((0, 0), (11, 1)):
        pg = int(table[r, far_key // page])
        for h in range(H):
            v = vc[pg, h // (H // K), far_key % page].float()
            torch.testing.assert_close(out.view(-1, H, d)[t_idx, h].float(), v, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_window_edge(ops, dtype):
    """A key that matches the query strongly lies just outside the window for one token and just
    inside it for the next: it must count for the second only."""
    g = torch.Generator(device=DEV).manual_seed(9)
    H, K, d, page, window = 2, 1, 32, 8, 50
    lens_new = [(100, 2)]          # queries at positions 100 and 101
    q, kc, vc, table, ctx = paged_case(g, dtype, lens_new, H, K, d, page, 16)
    kc.mul_(0.05)
    outside_for_101 = 51           # position 100 sees 51..100, position 101 sees 52..101
    key = torch.randn(d, device=DEV, generator=g)
    key = key / key.norm() * 6
    kc[int(table[0, outside_for_101 // page]), 0, outside_for_101 % page] = key.to(dtype)
    q.view(2, H, d)[:] = (key * 2).to(dtype)
    out, want = torch.empty_like(q), torch.empty_like(q)
    ops.attention(q, kc, vc, out, ctx, table, H, K, d, 1.0, window)
    ref.attention(q, kc, vc, want, ctx, table, H, K, d, 1.0, window)
    t = dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(out.float(), want.float(), **t)
    v = vc[int(table[0, outside_for_101 // page]), 0, outside_for_101 % page].float()
    torch.testing.assert_close(out.view(2, H, d)[0, 0].float(), v, rtol=2e-2, atol=2e-2)
    assert (out.view(2, H, d)[1, 0].float() - v).abs().max() > 0.1


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,I", [(1, 136), (7, 320), (33, 9728), (2, 3)])
def test_swiglu(ops, dtype, T, I):
    g = torch.Generator(device=DEV).manual_seed(10)
    gu = (torch.randn(T, 2 * I, device=DEV, generator=g) * 3).to(dtype)
    out, want = torch.empty(T, I, device=DEV, dtype=dtype), torch.empty(T, I, device=DEV, dtype=dtype)
    ops.swiglu(gu, out)
    ref.swiglu(gu, want)
    torch.testing.assert_close(out.float(), want.float(), **tol(dtype))


def test_gather_rows_add_into_argmax(ops):
    g = torch.Generator(device=DEV).manual_seed(11)
    src = torch.randn(50, 333, device=DEV, generator=g)
    rows = torch.tensor([49, 0, 7, 7, 31], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 333, device=DEV)
    ops.gather_rows(src, rows, out)
    assert torch.equal(out, src[rows.long()])
    for dtype in DTYPES:
        y = torch.randn(9, 77, device=DEV, generator=g)
        x = torch.randn(9, 77, device=DEV, generator=g).to(dtype)
        want = y + x.float()
        ops.add_into(y, x)
        assert torch.equal(y, want)
    logits = torch.randn(6, 151936, device=DEV, generator=g)
    logits[0, 5] = logits[0, 77777] = 50.0          # lowest id wins a tie
    logits[1, 151935] = 60.0                        # the last id
    logits[2, 151000] = 70.0                        # beyond `usable` below: must not be picked
    ids = torch.empty(6, dtype=torch.int32, device=DEV)
    ops.argmax(logits, 151936, ids)
    assert ids.tolist()[:2] == [5, 151935] and int(ids[2]) == 151000
    ops.argmax(logits, 150000, ids)
    assert ids.tolist() == torch.argmax(logits[:, :150000], dim=-1).tolist()


def test_kernels_refuse_what_they_cannot_do(ops):
    from marin_b200.kernels.ops import KernelError

    x = torch.zeros(4, 8)
    with pytest.raises(KernelError):
        ops.rmsnorm(x, torch.ones(8), 1e-6, torch.empty(4, 8))         # CPU tensors: no CPU path
    q = torch.zeros(1, 2 * 1024, device=DEV)
    kc = torch.zeros(2, 1, 16, 1024, device=DEV)
    ctx = SimpleNamespace(positions=torch.zeros(1, dtype=torch.int32, device=DEV), req_index=torch.zeros(1, dtype=torch.int32, device=DEV))
    with pytest.raises(KernelError):
        ops.attention(q, kc, kc, torch.empty_like(q), ctx, torch.zeros(1, 2, dtype=torch.int32, device=DEV), 2, 1, 1024, 1.0, 0)
    with pytest.raises(KernelError):
        ops.gemm(torch.zeros(2, 8, device=DEV, dtype=torch.float16), torch.zeros(2, 8, device=DEV, dtype=torch.float16), torch.zeros(2, 2, device=DEV, dtype=torch.float16))


TC_SHAPES = [(129, 2560, 4096), (300, 384, 1096), (1000, 1000, 200), (2048, 2560, 9728), (511, 6144, 2560),
             (1, 128, 64), (8, 6144, 2560), (8, 2560, 4096), (8, 2560, 9728), (64, 2560, 4096), (16, 300, 200), (17, 333, 136),
             (33, 1000, 72), (100, 257, 320), (200, 640, 1024), (2048, 1280, 2560), (300, 128, 8), (129, 129, 4104)]


@pytest.mark.parametrize("T,N,K", TC_SHAPES)
def test_gemm_tensor_cores(ops, T, N, K):
    """The tcgen05 kernel at decode shapes (split-K), prefill shapes and ragged edges in every dimension,
    against a float64 product of the same bf16 inputs.  Run twice: the split-K counters must be back at zero."""
    g = torch.Generator(device=DEV).manual_seed(13)
    x = torch.randn(T, K, device=DEV, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    # make rows and columns distinguishable beyond noise: a tile put in the wrong place shows
    x[:, 0] += torch.arange(T, device=DEV).to(torch.bfloat16) * 0.125
    w[:, 0] += (torch.arange(N, device=DEV) % 64).to(torch.bfloat16) * 0.0625
    want = x.double() @ w.double().t()
    scale = float(want.abs().max())
    for _ in range(2):
        out32 = torch.full((T, N), float("nan"), device=DEV)
        ops.gemm(x, w, out32)
        ops.check_device_errors()
        assert float((out32.double() - want).abs().max()) <= 2e-5 * scale + 1e-4
        out16 = torch.empty(T, N, device=DEV, dtype=torch.bfloat16)
        ops.gemm(x, w, out16)
        torch.testing.assert_close(out16.double(), want, rtol=1e-2, atol=1e-2 * scale)
        base = torch.randn(T, N, device=DEV, generator=g)
        acc = base.clone()
        ops.gemm(x, w, acc, accumulate=True)
        assert float((acc.double() - base.double() - want).abs().max()) <= 2e-5 * scale + 1e-4
    ops.check_device_errors()


@pytest.mark.parametrize("T,N,K", [(2048, 2560, 4096), (1000, 3000, 1032), (1999, 2560, 9728), (777, 6144, 72), (5000, 1152, 64), (600, 4864, 520)])
def test_gemm_stream_k(ops, monkeypatch, T, N, K):
    """Shapes for which the k-blocks, not the tiles, are dealt over the SMs: the pieces of a tile that two CTAs share
    must add up.  Against float64, against the tile-by-tile kernel, and twice (the flags must be back at zero).
    Column 0 of x and w carry ramps, and the first and the last k-block differ in size, so that a piece added
    to the wrong tile, added twice or left out shows."""
    monkeypatch.setattr(ops, "_STREAM_K_FIXED", -1e12)            # stream-K wherever it can run, not only where it pays
    assert ops.stream_k_plan(T, N, K) is not None
    g = torch.Generator(device=DEV).manual_seed(29)
    x = torch.randn(T, K, device=DEV, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    x[:, 0] += torch.arange(T, device=DEV).to(torch.bfloat16) * 0.125
    w[:, 0] += (torch.arange(N, device=DEV) % 64).to(torch.bfloat16) * 0.0625
    x[:, K - 1] += (torch.arange(T, device=DEV) % 7).to(torch.bfloat16)
    want = x.double() @ w.double().t()
    scale = float(want.abs().max())
    for _ in range(2):
        out32 = torch.full((T, N), float("nan"), device=DEV)
        ops.gemm(x, w, out32)
        ops.check_device_errors()
        assert float((out32.double() - want).abs().max()) <= 2e-5 * scale + 1e-4
        base = torch.randn(T, N, device=DEV, generator=g)
        acc = base.clone()
        ops.gemm(x, w, acc, accumulate=True)
        assert float((acc.double() - base.double() - want).abs().max()) <= 2e-5 * scale + 1e-4
        out16 = torch.empty(T, N, device=DEV, dtype=torch.bfloat16)
        ops.gemm(x, w, out16)
    ops.check_device_errors()
    monkeypatch.setattr(ops, "stream_k", False)
    plain16 = torch.empty_like(out16)
    ops.gemm(x, w, plain16)
    # float32 sums of the same products in another order, rounded to bf16: one step of bf16 apart at most
    torch.testing.assert_close(out16.float(), plain16.float(), rtol=2 ** -7, atol=1e-3 * scale)
    if N % 32 == 0:
        monkeypatch.setattr(ops, "stream_k", True)
        a = torch.empty(T, N // 2, device=DEV, dtype=torch.bfloat16)
        ops.gemm_swiglu(x, w, a)
        ops.check_device_errors()
        monkeypatch.setattr(ops, "stream_k", False)
        b = torch.empty_like(a)
        ops.gemm_swiglu(x, w, b)
        torch.testing.assert_close(a.float(), b.float(), rtol=2 ** -6, atol=1e-3 * scale * scale)


@pytest.mark.parametrize("T,N,K,N2,unit", [(8, 2560, 4096, 6144, False), (1, 320, 512, 384, False), (13, 200, 264, 96, True),
                                            (33, 1024, 9728, 2048, False), (64, 2560, 512, 640, False), (16, 128, 64, 64, True),
                                            (1000, 2560, 512, 2560, False), (2048, 2560, 1024, 6144, True), (777, 3072, 320, 96, False)])
def test_gemm_carries_the_norm_that_follows(ops, monkeypatch, T, N, K, N2, unit):
    """h += x W^T with the RMS norm of the new h riding on it, finished by the next product (plain and with
    SwiGLU): against float64, and against the same three steps with the norm as a kernel of its own."""
    g = torch.Generator(device=DEV).manual_seed(21)
    x = torch.randn(T, K, device=DEV, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    h0 = torch.randn(T, N, device=DEV, generator=g) * torch.linspace(0.2, 30.0, T, device=DEV)[:, None]   # rows of very different size
    gain = 1 + 0.2 * torch.randn(N, device=DEV, generator=g)
    w2 = (torch.randn(N2, N, device=DEV, generator=g) / math.sqrt(N)).to(torch.bfloat16)
    eps = 1e-5
    monkeypatch.setattr(ops, "COUPLED_NORM_MAX_TOKENS", 64)         # every tile width the kernel couples at
    monkeypatch.setattr(ops, "couple_norms_in_prefill", True)       # and the persistent kernel, for many tokens
    monkeypatch.setattr(ops, "stream_k", False)                     # the coupled product runs tile by tile: so must its twin, for equal bits
    for _ in range(2):
        h = h0.clone()
        normed = torch.full((T, N), float("nan"), device=DEV, dtype=torch.bfloat16)
        carried = ops.gemm(x, w, h, accumulate=True, then_norm=ops.NormOut(gain, unit, eps, normed))
        assert isinstance(carried, ops.NormedRows)
        want_h = h0.double() + x.double() @ w.double().t()
        assert float((h.double() - want_h).abs().max()) <= 2e-5 * float(want_h.abs().max()) + 1e-4
        y = torch.empty(T, N2, device=DEV, dtype=torch.bfloat16)
        ops.gemm(carried, w2, y)
        ops.check_device_errors()
        gg = (1 + gain.double()) if unit else gain.double()
        want_n = want_h / torch.sqrt((want_h ** 2).mean(dim=1, keepdim=True) + eps) * gg
        want_y = want_n @ w2.double().t()
        scale = float(want_y.abs().max())
        assert float((y.double() - want_y).abs().max()) <= 2e-2 * scale
        # the same with the norm as its own kernel
        h_b = h0.clone()
        ops.gemm(x, w, h_b, accumulate=True)
        n_b = torch.empty(T, N, device=DEV, dtype=torch.bfloat16)
        ops.rmsnorm(h_b, gain, eps, n_b, unit)
        y_b = torch.empty(T, N2, device=DEV, dtype=torch.bfloat16)
        ops.gemm(n_b, w2, y_b)
        assert torch.equal(h, h_b)
        assert float((y.float() - y_b.float()).abs().max()) <= 1.6e-2 * scale
        if N2 % 32 == 0:
            act, act_b = (torch.empty(T, N2 // 2, device=DEV, dtype=torch.bfloat16) for _ in range(2))
            ops.gemm_swiglu(carried, w2, act)
            ops.gemm_swiglu(n_b, w2, act_b)
            yy = want_y.float()
            blocks = yy.view(T, N2 // 32, 2, 16)
            gate, up = blocks[:, :, 0].reshape(T, -1), blocks[:, :, 1].reshape(T, -1)
            want_act = gate / (1 + torch.exp(-gate)) * up
            lim = 2e-2 * float(want_act.abs().max()) + 1e-3
            assert float((act.float() - want_act).abs().max()) <= lim
            assert float((act.float() - act_b.float()).abs().max()) <= lim
    ops.check_device_errors()


def test_gemm_with_many_tokens_leaves_the_norm_to_the_caller(ops):
    g = torch.Generator(device=DEV).manual_seed(22)
    x = torch.randn(200, 256, device=DEV, generator=g).to(torch.bfloat16)
    w = torch.randn(384, 256, device=DEV, generator=g).to(torch.bfloat16)
    h = torch.zeros(200, 384, device=DEV)
    normed = torch.empty(200, 384, device=DEV, dtype=torch.bfloat16)
    assert ops.gemm(x, w, h, accumulate=True, then_norm=ops.NormOut(torch.ones(384, device=DEV), False, 1e-6, normed)) is None
    assert float((h.double() - x.double() @ w.double().t()).abs().max()) <= 1e-2


@pytest.mark.parametrize("T,H,K,hidden,norm,rope,write", [(8, 32, 8, 2560, True, True, True), (1, 4, 2, 512, True, True, True),
                                                         (16, 6, 3, 1024, False, True, True), (5, 8, 1, 768, True, False, True),
                                                         (3, 4, 4, 512, True, True, False),
                                                         # up to 128 tokens: still the cluster's kernel
                                                         (64, 32, 8, 2560, True, True, True), (33, 6, 3, 1024, True, True, True),
                                                         (128, 32, 8, 2560, True, True, True), (100, 4, 2, 512, False, True, True),
                                                         (17, 8, 2, 768, True, False, False),
                                                         # many tokens: the persistent kernel, angles from the step's table
                                                         (2048, 32, 8, 2560, True, True, True), (300, 20, 5, 520, True, True, True),
                                                         (777, 12, 2, 1024, False, True, True), (1030, 9, 3, 768, True, False, True),
                                                         (500, 40, 8, 512, True, True, False)])
def test_qkv_product_finishes_its_heads(ops, T, H, K, hidden, norm, rope, write):
    """The q|k|v product with norm, rotation and cache write in its epilogue, against the product followed by the
    kernel that does the same on its own."""
    from types import SimpleNamespace

    from marin_b200.engine.context import Workspace

    d, page = 128, 16
    step = SimpleNamespace(extras={}, workspace=Workspace(DEV))
    g = torch.Generator(device=DEV).manual_seed(31)
    heads_total = H + 2 * K if write else H
    x = torch.randn(T, hidden, device=DEV, generator=g).to(torch.bfloat16)
    w = (torch.randn(heads_total * d, hidden, device=DEV, generator=g) / math.sqrt(hidden)).to(torch.bfloat16)
    w[:, 0] += (torch.arange(heads_total * d, device=DEV) % 128).to(torch.bfloat16) * 0.03       # rows distinguishable
    qw = (1 + 0.1 * torch.randn(d, device=DEV, generator=g)) if norm else None
    kw = (1 + 0.1 * torch.randn(d, device=DEV, generator=g)) if norm else None
    positions = torch.randint(0, 40000, (T,), device=DEV, generator=g, dtype=torch.int32)
    inv_freq = torch.pow(torch.tensor(1e6), -(torch.arange(d // 2, dtype=torch.float32) * 2.0 / d)).to(DEV) if rope else None
    pages = max(8, T // page + 3)
    slots = torch.randperm(pages * page, device=DEV, generator=g)[:T].to(torch.int32)
    if T > 2:
        slots[2] = -1
    if T > 200:
        slots[T - 1] = -1
    caches = [torch.zeros(pages, K, page, d, device=DEV, dtype=torch.bfloat16) for _ in range(4)]
    q1 = torch.full((T, H * d), float("nan"), device=DEV, dtype=torch.bfloat16)
    q2 = torch.empty_like(q1)
    for _ in range(2):
        done = ops.gemm_qkv_heads(x, w, q1, qw, kw, 1e-6, positions, inv_freq, d if rope else 0, False, slots, caches[0], caches[1],
                                  H, K, d, write, step)
        ops.check_device_errors()
        step.extras.clear()
    bn, splits = ops.gemm_plan(T, heads_total * d, hidden)
    assert done == (splits > 1 and T <= bn if T <= 128 else True)
    if not done:
        pytest.skip("this shape keeps K whole: no cluster to finish the heads in")
    qkv = torch.empty(T, heads_total * d, device=DEV, dtype=torch.bfloat16)
    # the twin's product goes to the kernel the fused one ran in (the persistent one from half a round of tiles on): the
    # sums then run in the same order, and a row that lands on a rounding boundary of bfloat16 rounds the same way
    rule = ops.many_tokens
    ops.many_tokens = lambda T_, N_, with_heads=False: rule(T_, N_, True)
    try:
        ops.gemm(x, w, qkv)
    finally:
        ops.many_tokens = rule
    ops.qk_norm_rope_write(qkv, q2, qw, kw, 1e-6, positions, inv_freq, d if rope else 0, False, slots, caches[2], caches[3], H, K, d, write)
    tol = dict(rtol=1.6e-2, atol=2e-2)
    torch.testing.assert_close(q1.float(), q2.float(), **tol)
    torch.testing.assert_close(caches[0].float(), caches[2].float(), **tol)
    torch.testing.assert_close(caches[1].float(), caches[3].float(), **tol)
    if write:
        assert float(caches[0].float().abs().sum()) > 0 and float(caches[1].float().abs().sum()) > 0


def test_qkv_product_declines_what_it_cannot_finish(ops):
    x = torch.zeros(40, 256, device=DEV, dtype=torch.bfloat16)
    w = torch.zeros(4 * 128, 256, device=DEV, dtype=torch.bfloat16)
    q = torch.zeros(40, 2 * 128, device=DEV, dtype=torch.bfloat16)
    cache = torch.zeros(4, 1, 16, 128, device=DEV, dtype=torch.bfloat16)
    slots = torch.zeros(40, device=DEV, dtype=torch.int32)
    assert not ops.gemm_qkv_heads(x, w, q, None, None, 1e-6, slots, None, 0, False, slots, cache, cache, 2, 1, 128, True)       # K stays whole: no cluster to meet in
    assert not ops.gemm_qkv_heads(x[:4], w[:, :], q[:4, :128].contiguous(), None, None, 1e-6, slots, None, 0, False, slots, cache,
                                  cache, 2, 1, 64, True)                                                                      # heads of 64


def test_gemm_tensor_cores_match_the_plain_kernel(ops):
    g = torch.Generator(device=DEV).manual_seed(14)
    x = torch.randn(40, 512, device=DEV, generator=g).to(torch.bfloat16)
    w = torch.randn(384, 512, device=DEV, generator=g).to(torch.bfloat16)
    a, b = torch.empty(40, 384, device=DEV), torch.empty(40, 384, device=DEV)
    ops.gemm(x, w, a)
    ops.use_tensor_cores = False
    try:
        ops.gemm(x, w, b)
    finally:
        ops.use_tensor_cores = True
    torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-3)


@pytest.mark.parametrize("H,K,d,page", [(32, 8, 128, 16), (8, 2, 64, 16), (6, 3, 48, 8), (40, 8, 128, 16)])
@pytest.mark.parametrize("window", [0, 300])
def test_attention_long_contexts_bf16(ops, H, K, d, page, window):
    """Several decode chunks and several query tiles per request, at the engine's page size."""
    g = torch.Generator(device=DEV).manual_seed(15)
    lens_new = [(1000, 1), (255, 1), (256, 1), (2049, 1), (900, 150), (0, 200), (511, 2)]
    pages = sum(-(-(c + n) // page) for c, n in lens_new) + 3
    q, kc, vc, table, ctx = paged_case(g, torch.bfloat16, lens_new, H, K, d, page, pages)
    out, want = torch.empty_like(q), torch.empty_like(q)
    ops.attention(q, kc, vc, out, ctx, table, H, K, d, 1.0 / math.sqrt(d), window)
    ref.attention(q, kc, vc, want, ctx, table, H, K, d, 1.0 / math.sqrt(d), window)
    torch.testing.assert_close(out.float(), want.float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("H,K,d,page", [(2, 2, 112, 64), (4, 4, 48, 16), (1, 1, 128, 16), (3, 3, 64, 16), (8, 2, 80, 8), (6, 2, 96, 32),
                                        (32, 8, 128, 16)])
def test_decode_chain_replayed_from_a_graph(ops, H, K, d, page):
    """The kernel that writes the new token's queries, keys and values and the decode attention behind it, captured
    in one graph and replayed over several positions.  Launched one by one the host's gaps keep kernels apart;
    replayed from a graph the attention really starts while its producer runs, and anything it reads too early (it
    asks for the older keys before it waits) is stale: the queries, keys and values change with every replay."""
    g = torch.Generator(device=DEV).manual_seed(41)
    B, first, steps = 3, [130, 17, 63], 7
    maxb = -(-(max(first) + steps + 1) // page) + 1
    pages = B * maxb + 2
    perm = torch.randperm(pages, generator=g, device=DEV)[: B * maxb].to(torch.int32).view(B, maxb)
    kc = torch.randn(pages, K, page, d, device=DEV, generator=g).to(torch.bfloat16)
    vc = torch.randn(pages, K, page, d, device=DEV, generator=g).to(torch.bfloat16)
    qw, kw = (1 + 0.1 * torch.randn(d, device=DEV, generator=g) for _ in range(2))
    inv_freq = (1e4 ** (-torch.arange(0, d, 2, device=DEV).float() / d)).contiguous()
    qkv = torch.zeros(B, (H + 2 * K) * d, device=DEV, dtype=torch.bfloat16)
    q = torch.zeros(B, H * d, device=DEV, dtype=torch.bfloat16)
    out = torch.zeros_like(q)
    positions = torch.zeros(B, dtype=torch.int32, device=DEV)
    slots = torch.zeros(B, dtype=torch.int32, device=DEV)
    ctx = SimpleNamespace(positions=positions, req_index=torch.arange(B, dtype=torch.int32, device=DEV),
                          cu_tokens=torch.arange(B + 1, dtype=torch.int32, device=DEV), seq_lens=torch.zeros(B, dtype=torch.int32, device=DEV),
                          num_tokens=B, num_requests=B, num_decode=B, max_query_len=1, max_seq_len=max(first) + steps + 1)
    plan = ops.DecodePlan(*ops.decode_split(B, K, 256))

    def chain():
        ops.qk_norm_rope_write(qkv, q, qw, kw, 1e-6, positions, inv_freq, d, False, slots, kc, vc, H, K, d)
        ops.attention(q, kc, vc, out, ctx, perm, H, K, d, 1.0 / math.sqrt(d), 0, plan)

    def set_step(i):
        pos = torch.tensor([f + i for f in first], dtype=torch.int32, device=DEV)
        positions.copy_(pos)
        ctx.seq_lens.copy_(pos + 1)
        page_of = perm[torch.arange(B, device=DEV), (pos // page).long()]
        slots.copy_(page_of * page + pos % page)
        qkv.copy_(torch.randn(qkv.shape, device=DEV, generator=g).to(torch.bfloat16))

    set_step(0)
    chain()                                              # builds what is needed before the capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        chain()
    for i in range(1, steps):
        set_step(i)
        graph.replay()
        torch.cuda.synchronize()
        ops.check_device_errors()
        want_q, want = torch.empty_like(q), torch.empty_like(out)
        kc2, vc2 = kc.clone(), vc.clone()
        ref.qk_norm_rope_write(qkv, want_q, qw, kw, 1e-6, positions, inv_freq, d, False, slots, kc2, vc2, H, K, d)
        torch.testing.assert_close(q.float(), want_q.float(), rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(kc.float(), kc2.float(), rtol=2e-2, atol=2e-2)
        ref.attention(want_q, kc2, vc2, want, ctx, perm, H, K, d, 1.0 / math.sqrt(d), 0)
        torch.testing.assert_close(out.float(), want.float(), rtol=3e-2, atol=3e-2, msg=lambda m: f"replay {i}: {m}")


@pytest.mark.parametrize("H,K,d,page,split,longest", [(32, 8, 128, 16, 128, 1500), (8, 2, 64, 16, 64, 1000), (4, 4, 48, 8, 64, 1023),
                                                      (5, 1, 128, 64, 64, 600)])
def test_attention_decode_in_clusters_of_more_than_eight(ops, H, K, d, page, split, longest):
    """Nine to sixteen chunks of a sequence are still one cluster where the device places clusters of that (non-portable)
    size, and merge through scratch memory where it does not: either way the result is the reference's."""
    g = torch.Generator(device=DEV).manual_seed(24)
    lens_new = [(longest, 1), (70, 1), (0, 1), (longest // 2, 1), (longest - 300, 1)]
    pages = sum(-(-(c + n) // page) for c, n in lens_new) + 2
    q, kc, vc, table, ctx = paged_case(g, torch.bfloat16, lens_new, H, K, d, page, pages)
    chunks = -(-(longest + 1) // split)
    assert 8 < chunks <= 16
    plan = ops.DecodePlan(split, chunks)
    want = torch.empty_like(q)
    ref.attention(q, kc, vc, want, ctx, table, H, K, d, 1.0 / math.sqrt(d), 0)
    for _ in range(2):
        out = torch.full_like(q, float("nan"))
        ops.attention(q, kc, vc, out, ctx, table, H, K, d, 1.0 / math.sqrt(d), 0, plan)
        ops.check_device_errors()
        torch.testing.assert_close(out.float(), want.float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("H,K,d,page,split", [(32, 8, 128, 16, 64), (8, 2, 64, 16, 64), (6, 3, 48, 8, 64), (4, 4, 128, 32, 64)])
def test_attention_decode_with_more_chunks_than_a_cluster_holds(ops, H, K, d, page, split):
    """Sequences cut into more chunks than a cluster holds merge through scratch memory (the last CTA combines them);
    run twice: the arrival counters must be back at zero."""
    g = torch.Generator(device=DEV).manual_seed(23)
    lens_new = [(1500, 1), (70, 1), (0, 1), (1023, 1), (640, 1)]
    pages = sum(-(-(c + n) // page) for c, n in lens_new) + 2
    q, kc, vc, table, ctx = paged_case(g, torch.bfloat16, lens_new, H, K, d, page, pages)
    chunks = -(-1501 // split)
    assert chunks > 16
    plan = ops.DecodePlan(split, chunks)
    want = torch.empty_like(q)
    ref.attention(q, kc, vc, want, ctx, table, H, K, d, 1.0 / math.sqrt(d), 0)
    for _ in range(2):
        out = torch.full_like(q, float("nan"))
        ops.attention(q, kc, vc, out, ctx, table, H, K, d, 1.0 / math.sqrt(d), 0, plan)
        ops.check_device_errors()
        torch.testing.assert_close(out.float(), want.float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("T,I,K", [(1, 9728, 2560), (8, 320, 96), (40, 144, 72), (300, 1024, 256), (2048, 2048, 512), (64, 4864, 1280)])
def test_gemm_with_swiglu_epilogue(ops, T, I, K):
    """silu(x Wg^T) * (x Wu^T) with the activation applied to the float32 accumulators, against float64."""
    g = torch.Generator(device=DEV).manual_seed(16)
    x = torch.randn(T, K, device=DEV, generator=g).to(torch.bfloat16)
    wg = (torch.randn(I, K, device=DEV, generator=g) / math.sqrt(K) * 2).to(torch.bfloat16)
    wu = (torch.randn(I, K, device=DEV, generator=g) / math.sqrt(K) * 2).to(torch.bfloat16)
    assert ops.can_fuse_swiglu(torch.bfloat16, K, I)
    w = ops.interleave_gate_up(wg, wu)
    out = torch.empty(T, I, device=DEV, dtype=torch.bfloat16)
    ops.gemm_swiglu(x, w, out)
    ops.check_device_errors()
    gd, ud = x.double() @ wg.double().t(), x.double() @ wu.double().t()
    want = gd / (1 + torch.exp(-gd)) * ud
    torch.testing.assert_close(out.double(), want, rtol=1e-2, atol=1e-2)
    # the two-kernel form gives the same up to the rounding of the intermediate
    ops.use_tensor_cores = False
    try:
        out2 = torch.empty_like(out)
        ops.gemm_swiglu(x, w, out2)
    finally:
        ops.use_tensor_cores = True
    torch.testing.assert_close(out2.double(), want, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("temperature,top_k,top_p", [(1.0, 0, 1.0), (0.7, 0, 0.9), (1.3, 5, 1.0), (0.5, 40, 0.6), (0.0, 0, 0.9), (2.0, 1, 1.0), (0.8, 300, 0.95)])
@pytest.mark.parametrize("vocab", [50, 2500])
def test_device_sampling_follows_the_reference_distribution(ops, temperature, top_k, top_p, vocab):
    """A grid of u values run through the device sampler: no token outside the host sampler's kept set is ever drawn,
    and the share of draws each kept token gets equals its probability (the host sampler is the reference's
    algorithm line by line).  Ties are planted at the head of the ranking."""
    from marin_b200.sampling import Sampler, SamplingParams

    g = torch.Generator(device=DEV).manual_seed(17)
    row = torch.randn(vocab, device=DEV, generator=g) * 2.0
    row[7] = row[3] = row.max() + 0.5                      # two equal best logits
    row[vocab - 1] = row[11]                               # a tie somewhere in the middle
    usable = vocab - 1                                     # the last id cannot be drawn
    N = 4000
    logits = row.unsqueeze(0).expand(N, vocab).contiguous()
    u = ((torch.arange(N, device=DEV, dtype=torch.float32) + 0.5) / N)
    out = torch.empty(N, dtype=torch.int32, device=DEV)
    ops.sample(logits, torch.full((N,), usable, dtype=torch.int32, device=DEV), torch.full((N,), temperature, device=DEV),
               torch.full((N,), top_k, dtype=torch.int32, device=DEV), torch.full((N,), top_p, device=DEV), u, out)
    counts = torch.bincount(out.long().cpu(), minlength=vocab).double() / N
    want = Sampler(SamplingParams(temperature=temperature, top_k=top_k, top_p=top_p)).distribution(row.cpu().numpy(), usable)
    probs = torch.zeros(vocab, dtype=torch.double)
    for token, p in want:
        probs[token] = p
    assert set(torch.nonzero(counts).flatten().tolist()) <= {t for t, _ in want}
    assert float((counts - probs).abs().max()) <= 2.0 / N + 1e-4
    if temperature == 0.0:
        assert int(out[0]) == 3 and bool((out == 3).all())       # the lower id of the two equal best


@pytest.mark.parametrize("H,K,d,page", [(32, 8, 128, 16), (8, 2, 64, 16), (5, 1, 64, 32), (40, 8, 128, 64)])
@pytest.mark.parametrize("window", [0, 300])
def test_attention_tensor_core_prefill_matches_the_mma_kernel(ops, H, K, d, page, window):
    """The tcgen05 prefill kernel against its plain twin and against the mma.sync kernel, on portions at several
    cached lengths, with ragged tile and block edges."""
    g = torch.Generator(device=DEV).manual_seed(18)
    lens_new = [(0, 1), (900, 150), (0, 200), (511, 2), (63, 129), (1000, 128), (17, 64)]
    pages = sum(-(-(c + n) // page) for c, n in lens_new) + 3
    q, kc, vc, table, ctx = paged_case(g, torch.bfloat16, lens_new, H, K, d, page, pages)
    got, mma, want = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
    scale = 1.0 / math.sqrt(d)
    ops.attention(q, kc, vc, got, ctx, table, H, K, d, scale, window)
    ops.check_device_errors()
    ops.use_tc_attention = False
    try:
        ops.attention(q, kc, vc, mma, ctx, table, H, K, d, scale, window)
    finally:
        ops.use_tc_attention = True
    ref.attention(q, kc, vc, want, ctx, table, H, K, d, scale, window)
    torch.testing.assert_close(mma.float(), want.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("H,K,d,page", [(8, 2, 128, 16), (4, 1, 64, 16), (6, 3, 128, 32)])
def test_attention_tensor_core_prefill_of_long_portions_against_the_plain_twin(ops, H, K, d, page):
    """The tcgen05 prefill kernel against the plain torch twin (not another kernel of the package) where a query tile
    walks many 64-key blocks: portions of 300 to 2,000 tokens over 0 to 2,048 cached ones, so that the running maximum
    moves and the accumulator is rescaled many times, and one portion behind 16,600 cached positions, whose keys lie on
    more pages than the kernel's page-id cache in shared memory holds (1,024; the rest is read from global memory).
    One key far back is made to stand out in each long request, so that a block skipped or weighted wrongly shows."""
    g = torch.Generator(device=DEV).manual_seed(29)
    lens_new = [(0, 2000), (2048, 300), (1500, 700), (0, 300)]
    if page == 16:
        lens_new.append((16600, 300))
    pages = sum(-(-(c + n) // page) for c, n in lens_new) + 3
    q, kc, vc, table, ctx = paged_case(g, torch.bfloat16, lens_new, H, K, d, page, pages)
    # in every request, the key at position 5 of kv head 0 gets the direction of that request's last query (head 0),
    # scaled so that its score towers over the others: the last rows must then return (nearly) that position's value
    starts = ctx.cu_tokens.tolist()
    for r in range(len(lens_new)):
        last = q[starts[r + 1] - 1, :d].float()
        page_id = int(table[r, 5 // page])
        kc[page_id, 0, 5 % page] = (last / last.norm() * 16.0).to(torch.bfloat16)
    got, want = torch.empty_like(q), torch.empty_like(q)
    scale = 1.0 / math.sqrt(d)
    ops.attention(q, kc, vc, got, ctx, table, H, K, d, scale, 0)
    ops.check_device_errors()
    ref.attention(q, kc, vc, want, ctx, table, H, K, d, scale, 0)
    torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)
    for r in range(len(lens_new)):
        row, page_id = starts[r + 1] - 1, int(table[r, 5 // page])
        weight_on_far_key = float((got[row, :d].float() * vc[page_id, 0, 5 % page].float()).sum() / (vc[page_id, 0, 5 % page].float() ** 2).sum())
        assert weight_on_far_key > 0.5, f"request {r}: the far key carries {weight_on_far_key:.2f} of the weight"


def test_sampling_kernels_mark_rows_that_are_not_finite(ops):
    """A NaN or an infinity among the usable logits of a row: arg-max and the sampler write the id -1 for that row
    (the reference refuses it: crates/sampler/src/lib.rs:135-137); rows beside it are untouched, a bad value beyond
    ``usable`` does not count, and the next launch finds the scratch clean."""
    g = torch.Generator(device=DEV).manual_seed(33)
    rows, vocab = 7, 50021
    logits = torch.randn(rows, vocab, device=DEV, generator=g)
    want = torch.argmax(logits[:, :50000], dim=-1).tolist()
    logits[1, 49999] = float("nan")                 # the last usable value, seen by the last block of the row
    logits[3, 0] = float("inf")                     # an infinity would win the comparison: it is refused all the same
    logits[4, 31000] = float("-inf")
    logits[5, 50010] = float("nan")                 # beyond usable: ignored
    ids = torch.full((rows,), -7, dtype=torch.int32, device=DEV)
    for _ in range(2):
        ops.argmax(logits, 50000, ids)
        got = ids.tolist()
        assert [got[i] for i in (1, 3, 4)] == [-1, -1, -1]
        assert [got[i] for i in (0, 2, 5, 6)] == [want[i] for i in (0, 2, 5, 6)]
    clean = torch.randn(rows, vocab, device=DEV, generator=g)
    ops.argmax(clean, 50000, ids)
    assert ids.tolist() == torch.argmax(clean[:, :50000], dim=-1).tolist()
    n = rows
    usable = torch.full((n,), 50000, dtype=torch.int32, device=DEV)
    temperature = torch.tensor([0.0, 0.8, 1.0, 0.0, 1.2, 0.7, 1.0], device=DEV)
    top_k = torch.tensor([0, 5, 0, 0, 40, 0, 3], dtype=torch.int32, device=DEV)
    top_p = torch.tensor([1.0, 0.9, 0.5, 1.0, 1.0, 0.9, 1.0], device=DEV)
    u = torch.full((n,), 0.37, device=DEV)
    ops.sample(logits, usable, temperature, top_k, top_p, u, ids)
    got = ids.tolist()
    assert [got[i] for i in (1, 3, 4)] == [-1, -1, -1] and got[0] == want[0] and all(0 <= got[i] < 50000 for i in (2, 5, 6))
    ops.check_device_errors()
