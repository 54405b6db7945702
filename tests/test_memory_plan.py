"""Memory planning on the host: the footprint is the sum of the parts' own figures, it is compared with a free-memory
figure given here (no GPU is asked), and what does not fit is refused with the numbers
(the reference: crates/model/src/qwen3/fit.rs:2-22, crates/model/src/qwen3/weight_bytes.rs:11-69)."""
import pytest
import torch

from helpers import CONFIGS, TINY_B, make_model_dir

GIB = 1 << 30


def build(raw):
    from marin_b200.config import Qwen3Config
    from marin_b200.engine import build_model

    return build_model(Qwen3Config.from_dict(raw))


def test_weight_bytes_are_what_the_loaded_tensors_hold(tmp_path):
    """The figure planned before loading equals the bytes of the tensors after loading, for a tied and an untied
    model, in both dtypes (norm weights are kept in float32, a tied head holds nothing of its own)."""
    from marin_b200.engine import load_model
    from marin_b200.parts import Runtime

    for name in ("A", "B"):
        for dtype in (torch.float32, torch.bfloat16):
            d = make_model_dir(str(tmp_path / f"{name}{dtype}"), CONFIGS[name], seed=1, dtype=dtype)
            _, model = load_model(d, Runtime(torch.device("cpu"), dtype))
            seen, held = set(), 0
            for part in model.parts():
                for value in vars(part).values():
                    if isinstance(value, torch.Tensor) and value.data_ptr() not in seen and value.numel() > 8:
                        seen.add(value.data_ptr())
                        held += value.numel() * value.element_size()
            assert model.weight_bytes(dtype) == held, (name, dtype)    # (a rotary table is made, not loaded, and is small)


def test_flops_and_bytes_read_of_the_qwen3_4b_layout():
    import bench

    model = build(bench.QWEN3_4B)
    h, inter, v, layers = 2560, 9728, 151936, 36
    per_layer = (32 * 128 + 2 * 8 * 128) * h + h * 32 * 128 + 3 * inter * h
    assert model.weight_bytes(torch.bfloat16) == 2 * (layers * per_layer + v * h) + 4 * (layers * (2 * h + 2 * 128) + h)
    # a decode step reads every layer, the head (the tied table), and only its own rows of the embedding
    read = model.bytes_read(8, torch.bfloat16)
    assert read == 2 * (layers * per_layer + v * h) + 4 * (layers * (2 * h + 2 * 128) + h) + 8 * h * 2
    assert model.cache_bytes_read(1, torch.bfloat16) == layers * 2 * 8 * 128 * 2
    T = 2048
    pairs = T * (T + 1) // 2
    assert model.flops(T, pairs, 1) == pytest.approx(2.0 * T * layers * per_layer + 4.0 * pairs * 32 * 128 * layers + 2.0 * v * h)


def test_pool_defaults_to_what_fits_and_too_much_is_refused_with_the_numbers():
    import bench
    from marin_b200.engine.memory import OutOfDeviceMemory, SLACK_BYTES, plan

    raw = dict(bench.QWEN3_14B)
    model = build(raw)
    dtype = torch.bfloat16
    weights = model.weight_bytes(dtype)
    assert 27 * GIB < weights < 29 * GIB
    # the whole window of 64 sequences of 40,960 positions is 400 GiB of cache: on a 180 GB device the pool is cut
    fp = plan(model, dtype, 16, 40960, 64, 2048, None, (1, 2, 4, 8, 16, 32, 64), free_bytes=178 * GIB)
    assert fp.pages_wanted == 64 * 2560 and fp.num_pages == fp.pages_that_fit < fp.pages_wanted
    assert fp.needed <= 178 * GIB and fp.needed + fp.page > 178 * GIB            # as many pages as fit, not one more
    assert fp.page == 40 * 16 * 2 * 8 * 128 * 2
    # a pool the caller asks for and that does not fit is an error that names the numbers and what would fit
    with pytest.raises(OutOfDeviceMemory) as err:
        plan(model, dtype, 16, 40960, 64, 2048, 64 * 2560, (), free_bytes=178 * GIB)
    text = str(err.value)
    would_fit = plan(model, dtype, 16, 40960, 64, 2048, None, (), free_bytes=178 * GIB).pages_that_fit
    assert "weights 27." in text and "cache 400.00 GiB" in text and "free 178.00 GiB" in text
    assert f"at most {would_fit} pages would fit" in text
    # weights alone too large: not even one sequence
    with pytest.raises(OutOfDeviceMemory, match="not even one sequence"):
        plan(model, dtype, 16, 40960, 64, 2048, None, (), free_bytes=28 * GIB)
    # plenty of room: the pool is what was wanted; the slack counts at the edge
    small = build(TINY_B)
    fp = plan(small, torch.float32, 8, 256, 4, 64, None, (), free_bytes=4 * GIB)
    assert fp.num_pages == fp.pages_wanted == 4 * 32 and fp.slack == SLACK_BYTES + 4 * GIB // 64
    edge = fp.needed - fp.slack + SLACK_BYTES            # with a slack given by the caller the edge is exact
    assert plan(small, torch.float32, 8, 256, 4, 64, 128, (), free_bytes=edge, slack=SLACK_BYTES).num_pages == 128
    with pytest.raises(OutOfDeviceMemory):
        plan(small, torch.float32, 8, 256, 4, 64, 128, (), free_bytes=edge - 1, slack=SLACK_BYTES)
    # nobody asked the device: the plan is made, nothing is refused
    assert plan(model, dtype, 16, 40960, 64, 2048, None, ()).num_pages == 64 * 2560


def test_a_toy_part_is_planned_from_its_own_figures():
    """Nothing in the planner knows attention: a mixer with a fixed-size state and matrices of its own is counted."""
    from marin_b200.parts import Mixer, StateNeed, TensorSpec

    class Decay(Mixer):
        def __init__(self):
            self.name = "m"

        def cache_need(self):
            return StateNeed((40,), torch.float32)

        def tensor_specs(self):
            return [TensorSpec("m.in.weight", (40, 40)), TensorSpec("m.gain", (40,), "norm")]

    m = Decay()
    assert m.weight_bytes(torch.bfloat16) == 40 * 40 * 2 + 40 * 4
    assert m.flops(3) == 2.0 * 3 * 40 * 40
    assert m.cache_need().bytes() == 160 and m.cache_need().bytes_read(1000, torch.bfloat16) == 160
    assert m.kernel_jobs(torch.bfloat16) == {} and m.decode_plan_key() is None and m.capturable
