"""The host-side choices of tile widths and splits (no GPU): whatever they pick must be a launch the kernels take."""
import pytest

from marin_b200.kernels import ops


@pytest.mark.parametrize("T", [129, 300, 512, 1000, 1024, 2048, 3000, 4096, 8192])
@pytest.mark.parametrize("N,K", [(6144, 2560), (2560, 4096), (19456, 2560), (2560, 9728), (7168, 5120), (5120, 17408), (384, 1096), (1152, 64)])
def test_stream_k_is_planned_only_where_the_kernel_takes_it(T, N, K):
    bn = ops.stream_k_plan(T, N, K)
    assert ops.persistent_plan(T, N) in ops.PERSISTENT_TILES
    if bn is None:
        return
    assert bn in ops.STREAM_K_TILES
    across, rows = -(-T // bn), -(-N // 128)
    groups = ops.SM_COUNT // across
    assert across <= ops.SM_COUNT and rows >= groups          # a tile is shared by two CTAs at most
    assert bn <= 256                                          # the parked tiles fit the scratch (sized for 256)


def test_stream_k_can_be_switched_off(monkeypatch):
    assert ops.stream_k_plan(2048, 2560, 9728) == 256
    monkeypatch.setattr(ops, "stream_k", False)
    assert ops.stream_k_plan(2048, 2560, 9728) is None


@pytest.mark.parametrize("T,N,K", [(1, 6144, 2560), (8, 2560, 9728), (16, 2560, 4096), (64, 151936, 2560), (128, 300, 200), (33, 1000, 72)])
def test_few_token_plan_keeps_every_slice_in_use(T, N, K):
    bn, splits = ops.gemm_plan(T, N, K)
    assert bn in (16, 32, 64, 128) and bn >= min(T, 128) and splits in (1, 2, 4, 8)
    nkb = -(-K // 64)
    per = -(-nkb // splits)
    assert (splits - 1) * per < nkb                            # no slice without k-blocks
