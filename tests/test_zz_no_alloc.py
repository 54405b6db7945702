"""mb_gemm_tc_noalloc, the matrix-product entry point for programs that may not allocate device memory
where the product runs (a process whose own arena owns the whole device, a latency-critical loop that
cannot afford cudaMalloc's device-wide stall, a plug-in under someone else's memory budget).  Its split-K
scratch is a fixed array inside the library, so the caller passes only inputs and outputs.

The test calls it through its exported C symbol, twice in a row (the scratch is shared between calls and
keeps what the last call left), and compares each result with the ordinary entry point's, at the
tolerance the other matrix-product tests use, and with a float64 product of the same inputs, so that the
check does not rest on another kernel of the same family.  Sizes beyond the built-in scratch must be refused with a
message, before anything is launched.  This file sorts last on purpose: a run that stops at the first
failure has then already run every other test.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def entry():
    from marin_b200.kernels import build

    lib = build.load("mb_gemm_tc", build.LIBRARIES["mb_gemm_tc"])
    fn = lib.mb_gemm_tc_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                   ctypes.c_int, ctypes.c_void_p]
    lib.mb_gemm_tc_noalloc_last_error.restype = ctypes.c_char_p
    lib.mb_gemm_tc_noalloc_device_error.restype = ctypes.c_int
    return lib, fn


@pytest.mark.parametrize("T,N,K", [(8, 2560, 4096), (5, 333, 1096), (64, 640, 2560), (300, 257, 320)])
def test_no_alloc_entry_matches_the_ordinary_one_twice_in_a_row(T, N, K):
    from marin_b200.kernels import ops

    lib, fn = entry()
    g = torch.Generator(device=DEV).manual_seed(21)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call in range(2):
        x = torch.randn(T, K, device=DEV, generator=g).to(torch.bfloat16)
        w = (torch.randn(N, K, device=DEV, generator=g) / math.sqrt(K)).to(torch.bfloat16)
        want32, want16 = torch.empty(T, N, device=DEV), torch.empty(T, N, device=DEV, dtype=torch.bfloat16)
        ops.gemm(x, w, want32)
        ops.gemm(x, w, want16)
        got32 = torch.full((T, N), float("nan"), device=DEV)
        got16 = torch.empty(T, N, device=DEV, dtype=torch.bfloat16)
        assert fn(x.data_ptr(), w.data_ptr(), got32.data_ptr(), 1, T, N, K, stream) == 0, lib.mb_gemm_tc_noalloc_last_error()
        assert fn(x.data_ptr(), w.data_ptr(), got16.data_ptr(), 0, T, N, K, stream) == 0
        base = torch.randn(T, N, device=DEV, generator=g)
        acc = base.clone()
        assert fn(x.data_ptr(), w.data_ptr(), acc.data_ptr(), 2, T, N, K, stream) == 0
        torch.cuda.synchronize()
        scale = float(want32.abs().max())
        assert float((got32 - want32).abs().max()) <= 2e-5 * scale + 1e-4, f"call {call}"
        exact = x.double() @ w.double().t()                  # bfloat16 products are exact in float64: only the sums round
        assert float((got32.double() - exact).abs().max()) <= 2e-5 * scale + 1e-4, f"call {call} against float64"
        torch.testing.assert_close(got16.float(), want16.float(), rtol=1e-2, atol=1e-2 * scale)
        assert float((acc - base - want32).abs().max()) <= 2e-5 * scale + 1e-4
    assert lib.mb_gemm_tc_noalloc_device_error() == 0


def test_no_alloc_entry_on_a_stream_of_the_callers_own():
    """Callers run the product on streams of their own, which do not wait for the legacy default stream nor it for
    them.  The flag reader has to wait for the whole device by itself: here nothing synchronises before it is
    called, and afterwards the result is complete and right."""
    lib, fn = entry()
    g = torch.Generator(device=DEV).manual_seed(22)
    T, N, K = 8, 2560, 4096
    x = torch.randn(T, K, device=DEV, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device=DEV, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    exact = x.double() @ w.double().t()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    got = torch.full((T, N), float("nan"), device=DEV)
    with torch.cuda.stream(side):
        for _ in range(3):
            assert fn(x.data_ptr(), w.data_ptr(), got.data_ptr(), 1, T, N, K, ctypes.c_void_p(side.cuda_stream)) == 0
    assert lib.mb_gemm_tc_noalloc_device_error() == 0         # waits for the side stream too
    assert side.query()                                       # ... so nothing is left running on it
    assert float((got.double() - exact).abs().max()) <= 2e-5 * float(exact.abs().max()) + 1e-4


def test_no_alloc_entry_refuses_what_its_scratch_cannot_hold():
    lib, fn = entry()
    x = torch.zeros(128, 8192, device=DEV, dtype=torch.bfloat16)
    w = torch.zeros(2048, 8192, device=DEV, dtype=torch.bfloat16)
    out = torch.full((128, 2048), 7.0, device=DEV)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # 16 tiles -> 16 K slices x 128 x 2048 floats = 4 Mi floats: twice what the built-in scratch holds
    rc = fn(x.data_ptr(), w.data_ptr(), out.data_ptr(), 1, 128, 2048, 8192, stream)
    assert rc == -5
    text = lib.mb_gemm_tc_noalloc_last_error().decode()
    assert "scratch" in text and "2097152" in text and "4194304" in text
    torch.cuda.synchronize()
    assert float(out.min()) == 7.0                      # nothing was launched
    assert fn(x.data_ptr(), w.data_ptr(), out.data_ptr(), 1, 128, 2048, 7, stream) == -3      # K not a multiple of 8
