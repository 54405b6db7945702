"""The engine at the layer sizes of real models and at real batch sizes, against the plain implementation.

One layer with every width of the Qwen3-4B, 8B and 14B layouts (hidden size, head counts, head size,
intermediate size; the vocabulary is cut to 8,200 rows and the model to one layer so that the plain
implementation, on the CPU, stays in seconds), a context above 1,024, in float32 and in bfloat16, under every
way of cutting the work: whole; all but the last 32 tokens in one step and those one by one from graphs;
portions of changing size down to two tokens; five requests mixed four at a time in a pool so small that pages
are used again.  These sizes reach the code the tiny configurations never do: the persistent and stream-K
matrix products, cluster split-K at real K, the tcgen05 attention over many key blocks, the TMA decode kernel.

And many live requests: 8, 20 and 64 requests decoding together (graph buckets 8, 32 and 64, rows that pad a
batch, token tiles of 16, 32 and 64, norms that no longer ride on products, other splits of the keys) on a tiny
configuration with heads of 128 and on the 4B-width layer, every row of logits against the plain implementation.

The comparison the reference makes at its own sizes: crates/model/tests/kv_append.rs:27-60 (chunked against whole).
"""
import math
import random

import pytest
import torch

import plain_qwen3 as plain
from helpers import CONFIGS, MATRIX_STD, PAGE, make_model_dir, mixed_schedule, portions, random_prompt, run_mixed, run_portions, run_whole
from test_engine_gpu import close, plain_forward

pytestmark = pytest.mark.gpu

VOCAB = 8200
BASE = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 1, "head_dim": 128,
        "num_key_value_heads": 8, "vocab_size": VOCAB, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "max_position_embeddings": 2048}
LAYOUTS = {
    "4b": dict(BASE, hidden_size=2560, num_attention_heads=32, intermediate_size=9728, tie_word_embeddings=True),
    "8b": dict(BASE, hidden_size=4096, num_attention_heads=32, intermediate_size=12288, tie_word_embeddings=False),
    "14b": dict(BASE, hidden_size=5120, num_attention_heads=40, intermediate_size=17408, tie_word_embeddings=False),
}
LENGTHS = {"a": 1100, "b": 400, "c": 130, "d": 700, "e": 250}
PAGE_SIZE = 16


class Layout:
    """One layer of a layout: the folder (bfloat16 weights: the float32 engine reads the same values, so one plain
    result serves both dtypes), the plain logits, and engines' parts per dtype."""

    def __init__(self, tmp, name):
        raw = LAYOUTS[name]
        self.name, self.raw = name, raw
        # matrices of standard deviation 1 / sqrt(width): logits of standard deviation about 1, which the tolerances suppose
        self.dir = make_model_dir(str(tmp / name), raw, seed=21, dtype=torch.bfloat16, matrix_std=1.0 / math.sqrt(raw["hidden_size"]))
        self.cfg, self.w = plain.read_config(self.dir), plain.read_weights(self.dir)
        rng = random.Random(17)
        self.tokens = {rid: random_prompt(rng, VOCAB, n) for rid, n in LENGTHS.items()}
        self.wanted = {}
        self.models = {}

    def want(self, dtype):
        """The plain logits of the five requests as an engine of this dtype should reproduce them (bfloat16: rounded
        where a 16-bit engine stores activations), computed when first asked for."""
        if dtype not in self.wanted:
            self.wanted[dtype] = {rid: plain_forward(self.cfg, self.w, t, dtype) for rid, t in self.tokens.items()}
        return self.wanted[dtype]

    def model(self, dtype):
        from marin_b200.engine import load_model, parse_dtype
        from marin_b200.parts import Runtime

        if dtype not in self.models:
            rt = Runtime(torch.device("cuda:0"), parse_dtype(dtype))
            self.models[dtype] = (rt, load_model(self.dir, rt)[1])
        return self.models[dtype]

    def runner(self, dtype, num_pages, max_requests=4, graphs=(1, 2, 4)):
        from marin_b200.cache import CacheManager
        from marin_b200.engine import Runner

        rt, model = self.model(dtype)
        cache = CacheManager(model.cache_needs(), [e.cache_of for e in model.spec.schedule], PAGE_SIZE, num_pages, max_requests)
        cache.allocate(rt.device, rt.dtype)
        runner = Runner(model, cache, rt, self.raw["max_position_embeddings"])
        if graphs:
            runner.enable_graphs(graphs)
        return runner


_LAYOUTS = {}


def layout_of(name, tmp_path_factory) -> Layout:
    if name not in _LAYOUTS:
        _LAYOUTS[name] = Layout(tmp_path_factory.mktemp("layouts"), name)
    return _LAYOUTS[name]


@pytest.fixture(scope="module", autouse=True)
def forget_layouts():
    yield
    _LAYOUTS.clear()              # the models' device memory goes back when the module is done
    torch.cuda.empty_cache()


@pytest.fixture(scope="module", params=["4b", "8b", "14b"])
def layout(request, tmp_path_factory):
    return layout_of(request.param, tmp_path_factory)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_way_of_cutting_at_real_widths(layout, dtype):
    wanted = layout.want(dtype)
    assert abs(float(wanted["a"].std()) - 1.0) < 0.35
    toks, want = layout.tokens["a"], wanted["a"]
    n = len(toks)
    runner = layout.runner(dtype, num_pages=-(-n // PAGE_SIZE) + 1)
    whole = run_whole(runner, "w", toks)
    close(whole, want, dtype, "whole")
    tail = run_portions(runner, "t", toks, [n - 32] + [1] * 32)
    close(tail, want, dtype, "tail of 32 decoded from graphs")
    assert any(g["graph"] is not None for g in runner.graphs.values())
    cut = run_portions(runner, "p", toks, portions(n, [300, 2, 500, 3, 2, 129, 64]))
    close(cut, want, dtype, "portions")
    runner.cache.check()
    need = sorted((-(-m // PAGE_SIZE) for m in LENGTHS.values()), reverse=True)
    runner = layout.runner(dtype, num_pages=sum(need[:4]))              # four live requests fit only through reuse
    steps = mixed_schedule(random.Random(3), LENGTHS, max_live=4, decode_tail=9, sizes=(260, 2, 410, 3, 2, 150))
    assert any(any(c == 1 for _, c in e) and any(c > 128 for _, c in e) for e, _ in steps)
    got = run_mixed(runner, layout.tokens, steps)
    for rid in LENGTHS:
        close(got[rid], wanted[rid], dtype, f"mixed {rid}")
    runner.cache.check()
    runner.scratch.check()
    if dtype == "float32":
        # the 32-bit path sums every product in one fixed order per output value: how the work was cut must not
        # show in a single bit
        assert torch.equal(whole, tail) and torch.equal(whole, cut) and torch.equal(whole, got["a"])


# ---- many live requests --------------------------------------------------------------------------------------------------

def decode_together(runner, tokens, prompt_len, budget=512):
    """Feeds every request's prompt (several requests a step, under a token budget), then lets all of them decode
    together, one token each per step, until each has been fed whole; requests of different lengths end at different
    steps, so the batch shrinks through every size.  Returns each request's logits at every position and the
    sizes of the single-token batches that ran."""
    from marin_b200.engine import StepEntry

    rows = {rid: [] for rid in tokens}
    fed = {rid: 0 for rid in tokens}
    waiting = list(tokens)
    batch, used = [], 0
    while waiting or batch:
        if waiting and used + prompt_len[waiting[0]] <= budget:
            rid = waiting.pop(0)
            runner.begin(rid)
            batch.append(rid)
            used += prompt_len[rid]
            continue
        logits = runner.step([StepEntry(rid, tokens[rid][:prompt_len[rid]], list(range(prompt_len[rid]))) for rid in batch]).clone()
        at = 0
        for rid in batch:
            rows[rid].append(logits[at:at + prompt_len[rid]])
            at += prompt_len[rid]
            fed[rid] = prompt_len[rid]
        batch, used = [], 0
    sizes = []
    live = [rid for rid in tokens if fed[rid] < len(tokens[rid])]
    for rid in tokens:
        if rid not in live:
            runner.end(rid)
    while live:
        logits = runner.step([StepEntry(rid, [tokens[rid][fed[rid]]], [0]) for rid in live]).clone()
        sizes.append(len(live))
        for i, rid in enumerate(live):
            rows[rid].append(logits[i:i + 1])
            fed[rid] += 1
        for rid in [r for r in live if fed[r] == len(tokens[r])]:
            runner.end(rid)
            live.remove(rid)
    return {rid: torch.cat(r) for rid, r in rows.items()}, sizes


def many_requests(rng, vocab, count, longest):
    """``count`` requests: prompts of 1 to about two thirds of ``longest`` tokens, then 6 to 40 decoded ones."""
    tokens, prompt_len = {}, {}
    for i in range(count):
        p = rng.randrange(1, max(2, longest * 2 // 3))
        total = min(longest, p + rng.randrange(6, 41))
        tokens[f"r{i}"] = random_prompt(rng, vocab, total)
        prompt_len[f"r{i}"] = p
    return tokens, prompt_len


@pytest.mark.parametrize("live", [8, 20, 64])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_many_requests_decoding_together_on_the_tiny_configuration_with_heads_of_128(tmp_path_factory, dtype, live):
    from marin_b200.cache import CacheManager
    from marin_b200.engine import Runner, load_model, parse_dtype
    from marin_b200.parts import Runtime

    raw = CONFIGS["D"]
    d = make_model_dir(str(tmp_path_factory.mktemp("many") / "D"), raw, seed=13, dtype=parse_dtype(dtype), matrix_std=MATRIX_STD["D"])
    cfg, w = plain.read_config(d), plain.read_weights(d)
    rt = Runtime(torch.device("cuda:0"), parse_dtype(dtype))
    _, model = load_model(d, rt)
    tokens, prompt_len = many_requests(random.Random(live), raw["vocab_size"], live, raw["max_position_embeddings"])
    pages = sum(-(-len(t) // PAGE["D"]) for t in tokens.values())
    cache = CacheManager(model.cache_needs(), [e.cache_of for e in model.spec.schedule], PAGE["D"], pages, live)
    cache.allocate(rt.device, rt.dtype)
    runner = Runner(model, cache, rt, raw["max_position_embeddings"])
    runner.enable_graphs((1, 2, 4, 8, 16, 32, 64))
    got, sizes = decode_together(runner, tokens, prompt_len)
    assert max(sizes) == live and {b for b, _ in runner.graphs} >= {next(b for b in (8, 32, 64) if b >= live)}
    for rid, toks in tokens.items():
        close(got[rid], plain_forward(cfg, w, toks, dtype), dtype, f"{live} live, request {rid} ({prompt_len[rid]} + {len(toks) - prompt_len[rid]})")
    cache.check()
    runner.scratch.check()
    assert not cache.requests


@pytest.mark.parametrize("live", [8, 20, 64])
def test_many_requests_decoding_together_at_4b_widths(tmp_path_factory, live):
    """bfloat16 only: it is the 16-bit kernels whose choices change with the batch size (the float32 kernels are the
    same at every size and are held to it on the tiny configuration above)."""
    layout = layout_of("4b", tmp_path_factory)
    tokens, prompt_len = many_requests(random.Random(100 + live), VOCAB, live, 160)
    pages = sum(-(-len(t) // PAGE_SIZE) for t in tokens.values())
    runner = layout.runner("bfloat16", pages, max_requests=live, graphs=(1, 2, 4, 8, 16, 32, 64))
    got, sizes = decode_together(runner, tokens, prompt_len, budget=1024)
    assert max(sizes) == live
    for rid, toks in tokens.items():
        close(got[rid], plain_forward(layout.cfg, layout.w, toks, "bfloat16"), "bfloat16", f"{live} live, request {rid}")
    runner.cache.check()
    runner.scratch.check()
