"""Configurations drawn at random (head sizes in steps of 16 and beyond 128, any number of heads and groups, widths and
vocabularies that are no power of two, every page size) through the step function in float32 and in bfloat16,
whole, with a decoded tail and in changing portions, against the plain implementation.  The kernels must take every
size the configuration allows, through a fused path or a plain one, and never give a wrong result."""
import random

import pytest
import torch

import plain_qwen3 as plain
from helpers import make_model_dir, portions, random_prompt, run_portions, run_whole
from test_engine_gpu import close, plain_forward

pytestmark = pytest.mark.gpu


def draw(rng: random.Random) -> tuple:
    d = rng.choice([16, 32, 48, 64, 80, 96, 112, 128, 128, 160, 256])
    kv = rng.choice([1, 2, 3, 4])
    heads = kv * rng.choice([1, 2, 3, 4, 5, 7, 8, 10])
    hidden = rng.choice([40, 72, 96, 136, 200, 264, 512, 520, 776])
    raw = {"model_type": "qwen3", "num_hidden_layers": rng.choice([1, 2, 3]), "hidden_size": hidden,
           "num_attention_heads": heads, "num_key_value_heads": kv, "head_dim": d,
           "intermediate_size": rng.choice([48, 80, 144, 176, 272, 640, 1000]), "vocab_size": rng.choice([97, 300, 333, 1001]),
           "rope_theta": rng.choice([1e4, 1e6]), "rms_norm_eps": rng.choice([1e-6, 1e-5]),
           "tie_word_embeddings": rng.random() < 0.5, "max_position_embeddings": 200}
    return raw, rng.choice([2, 4, 8, 16, 16, 32, 64]), rng.choice([37, 70, 130, 190])


#: Configurations that once went wrong.  One query head per kv head with heads that are not 128 wide, decoded from
#: graphs: the compiler had moved the loads of the queries above the wait for the kernel that writes them (it showed
#: only in graphs, where kernels really overlap, and only in the build for groups of one).
PINNED = [
    ({"model_type": "qwen3", "num_hidden_layers": 1, "hidden_size": 136, "num_attention_heads": 2, "num_key_value_heads": 2,
      "head_dim": 112, "intermediate_size": 48, "vocab_size": 300, "rope_theta": 1e4, "rms_norm_eps": 1e-5,
      "tie_word_embeddings": True, "max_position_embeddings": 200}, 64, 37),
    ({"model_type": "qwen3", "num_hidden_layers": 2, "hidden_size": 200, "num_attention_heads": 4, "num_key_value_heads": 4,
      "head_dim": 48, "intermediate_size": 144, "vocab_size": 333, "rope_theta": 1e6, "rms_norm_eps": 1e-6,
      "tie_word_embeddings": False, "max_position_embeddings": 200}, 16, 130),
]


@pytest.mark.parametrize("seed", list(range(6)) + [f"pinned{i}" for i in range(len(PINNED))])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_random_configuration(tmp_path, seed, dtype):
    from marin_b200.cache import CacheManager
    from marin_b200.engine import Runner, load_model, parse_dtype
    from marin_b200.kernels import ops
    from marin_b200.parts import Runtime

    if isinstance(seed, str):
        raw, page, n = PINNED[int(seed[len("pinned"):])]
        seed = 26
        rng = random.Random(3)
    else:
        rng = random.Random(100 + seed)
        raw, page, n = draw(rng)
    std = min(0.1, 1.2 / raw["hidden_size"] ** 0.5)              # logits of standard deviation near 1
    folder = make_model_dir(str(tmp_path / "m"), raw, seed=seed, dtype=parse_dtype(dtype), matrix_std=std)
    cfg, w = plain.read_config(folder), plain.read_weights(folder)
    rt = Runtime(torch.device("cuda:0"), parse_dtype(dtype))
    _, model = load_model(folder, rt)
    toks = random_prompt(rng, raw["vocab_size"], n)
    want = plain_forward(cfg, w, toks, dtype)
    cache = CacheManager(model.cache_needs(), [e.cache_of for e in model.spec.schedule], page, -(-200 // page) * 2, 4)
    cache.allocate(rt.device, rt.dtype)
    runner = Runner(model, cache, rt, 200)
    runner.enable_graphs((1, 2))
    what = f"{raw} page {page}"
    close(run_whole(runner, "w", toks), want, dtype, f"whole, {what}")
    tail = min(20, n - 1)
    close(run_portions(runner, "t", toks, [n - tail] + [1] * tail), want, dtype, f"decoded tail, {what}")
    close(run_portions(runner, "p", toks, portions(n, [7, 2, 13, 3, 2, 5, 64])), want, dtype, f"portions, {what}")
    ops.check_device_errors()
    cache.check()
