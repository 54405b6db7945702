"""The engine's host logic (flattening, block tables, page reuse, commits) with the CUDA kernels
replaced by their plain torch twins, so that it runs without a GPU.  The GPU tests repeat these
comparisons with the real kernels."""
import random

import pytest
import torch

import plain_qwen3 as plain
from helpers import CONFIGS, PAGE, make_model_dir, mixed_schedule, portions, random_prompt, run_mixed, run_portions, run_whole
from kernel_refs import patch_ops


def cpu_runner(model_dir, page_size, num_pages, max_requests=4, max_seq_len=None):
    from marin_b200.cache import CacheManager
    from marin_b200.engine import Runner, load_model
    from marin_b200.parts import Runtime

    rt = Runtime(torch.device("cpu"), torch.float32)
    config, model = load_model(model_dir, rt)
    cache = CacheManager(model.cache_needs(), [e.cache_of for e in model.spec.schedule], page_size, num_pages, max_requests)
    cache.allocate(rt.device, rt.dtype)
    return config, Runner(model, cache, rt, max_seq_len or config.max_position_embeddings)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_portions_and_mixed_equal_plain(tmp_path, name):
    raw = CONFIGS[name]
    d = make_model_dir(str(tmp_path / name), raw, seed=11, dtype=torch.float32, matrix_std=0.1)
    cfg, w = plain.read_config(d), plain.read_weights(d)
    rng = random.Random(5)
    lengths = {"a": 37, "b": 9, "c": 52, "d": 1, "e": 23, "f": 40}
    tokens = {rid: random_prompt(rng, raw["vocab_size"], n) for rid, n in lengths.items()}
    want = {rid: plain.forward(cfg, w, t) for rid, t in tokens.items()}
    page = PAGE[name]
    with patch_ops():
        # so few pages that four live requests fit only because finished ones give theirs back
        need = sorted((-(-n // page) for n in lengths.values()), reverse=True)
        config, runner = cpu_runner(d, page, num_pages=sum(need[:4]))
        for rid in ("a", "c"):
            got = run_whole(runner, rid, tokens[rid])
            torch.testing.assert_close(got, want[rid], rtol=1e-4, atol=1e-5)
            got = run_portions(runner, rid, tokens[rid], portions(len(tokens[rid]), [7, 2, 13, 3, 2]))
            torch.testing.assert_close(got, want[rid], rtol=1e-4, atol=1e-5)
        steps = mixed_schedule(rng, lengths)
        got = run_mixed(runner, tokens, steps)
        for rid in tokens:
            torch.testing.assert_close(got[rid], want[rid], rtol=1e-4, atol=1e-5)
        runner.cache.check()
        assert not runner.cache.requests
        assert all(g.pool.num_held == 0 for g in runner.cache.groups)


def test_failed_step_commits_nothing(tmp_path):
    from marin_b200.cache import OutOfPages
    from marin_b200.engine import StepEntry, StepError

    d = make_model_dir(str(tmp_path / "A"), CONFIGS["A"], seed=3)
    with patch_ops():
        config, runner = cpu_runner(d, 4, num_pages=4, max_seq_len=32)
        runner.begin("x")
        runner.step([StepEntry("x", [1, 2, 3, 4, 5], [4])])
        with pytest.raises(StepError):
            runner.step([StepEntry("x", [1, 999], [])])          # id outside the vocabulary
        with pytest.raises(OutOfPages):
            runner.step([StepEntry("x", list(range(12)), [])])   # 17 positions need 5 pages, 4 exist
        with pytest.raises(StepError):
            runner.step([StepEntry("x", list(range(40)), [])])   # beyond the context
        assert runner.length("x") == 5
        runner.cache.check()
        runner.end("x")
        runner.cache.check()
