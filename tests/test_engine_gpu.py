"""The engine on the GPU against the plain implementation, in 32-bit and in bfloat16, under every
way of cutting the work: each request alone and whole; most of it in one step and the last 32
tokens one by one; portions of changing size down to two tokens; and mixed batches of up to four
live requests with so few pages that they are used again.  Also long decoding, the first tokens of
a sequence and greedy generation through the entry point.

Tolerances (fixed; the reference's chunking gate is 1e-4 (1 + |x|), crates/model/tests/kv_append.rs:27-60):
float32: |diff| <= 1e-4 + 1e-4 |ref|.  bfloat16 (logits of standard deviation ~1): max |diff| <= 0.08 and
mean |diff| <= 0.01 against the plain implementation computed from the same bfloat16 weights and rounded to
bfloat16 where a 16-bit engine stores its activations (``plain.forward(..., stored=plain.as_bf16)``).  Measured
on B200 over the four tiny configurations and one layer of the Qwen3-4B, 8B and 14B widths, in every way of
cutting: max 0.025 to 0.046, mean 0.003 to 0.0063 (against the unrounded plain result: max up to 0.063, mean
up to 0.0081).  The rounded oracle takes out the part of the difference that is the same rounding on both sides;
what is left is rounding that falls differently because sums run in another order and factors are applied at
another place (a norm's factor after the product instead of before, softmax terms against a running maximum).
"""
import random

import pytest
import torch

import plain_qwen3 as plain
from helpers import MATRIX_STD, CONFIGS, PAGE, make_model_dir, mixed_schedule, portions, random_prompt, run_mixed, run_portions, run_whole

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
LENGTHS = {"A": {"a": 37, "b": 9, "c": 120, "d": 1, "e": 64, "f": 40, "g": 33},
           "B": {"a": 100, "b": 1, "c": 250, "d": 17, "e": 64, "f": 129, "g": 48},
           "C": {"a": 50, "b": 180, "c": 16, "d": 97, "e": 2, "f": 33},
           "D": {"a": 150, "b": 21, "c": 64, "d": 3, "e": 129, "f": 40}}


BF16_MAX, BF16_MEAN = 0.08, 0.01


def plain_forward(cfg, w, tokens, dtype: str, **kw):
    """The plain implementation's logits as the engine of this dtype should reproduce them."""
    return plain.forward(cfg, w, tokens, stored=plain.as_bf16 if dtype == "bfloat16" else plain.same, **kw)


def close(got: torch.Tensor, want: torch.Tensor, dtype: str, what=""):
    got, want = got.float().cpu(), want.float()
    assert got.shape == want.shape, (got.shape, want.shape)
    err = (got - want).abs()
    if dtype == "float32":
        bad = err > 1e-4 + 1e-4 * want.abs()
        if bad.any():
            first = int(torch.nonzero(bad.any(dim=1))[0])
            raise AssertionError(f"{what}: first wrong position {first} of {got.shape[0]}, max err {err.max():.3e}")
    else:
        rowmax = err.max(dim=1).values
        if err.max() > BF16_MAX or err.mean() > BF16_MEAN:
            first = int(torch.nonzero(rowmax > BF16_MAX)[0]) if (rowmax > BF16_MAX).any() else -1
            raise AssertionError(f"{what}: max err {err.max():.3e} mean {err.mean():.3e}, first position over the limit {first}")


class Case:
    def __init__(self, tmp, name, dtype):
        from marin_b200.cache import CacheManager
        from marin_b200.engine import Runner, load_model, parse_dtype
        from marin_b200.parts import Runtime

        raw = CONFIGS[name]
        self.name, self.dtype, self.raw = name, dtype, raw
        self.dir = make_model_dir(str(tmp / f"{name}-{dtype}"), raw, seed=11, dtype=parse_dtype(dtype), matrix_std=MATRIX_STD[name])
        self.cfg, self.w = plain.read_config(self.dir), plain.read_weights(self.dir)
        rng = random.Random(5)
        self.tokens = {rid: random_prompt(rng, raw["vocab_size"], n) for rid, n in LENGTHS[name].items()}
        self.want = {rid: plain_forward(self.cfg, self.w, t, dtype) for rid, t in self.tokens.items()}
        self.rt = Runtime(torch.device("cuda:0"), parse_dtype(dtype))
        self.config, self.model = load_model(self.dir, self.rt)
        self.page = PAGE[name]

    def runner(self, num_pages, max_requests=4, graphs=False):
        from marin_b200.cache import CacheManager
        from marin_b200.engine import Runner

        cache = CacheManager(self.model.cache_needs(), [e.cache_of for e in self.model.spec.schedule], self.page,
                             num_pages, max_requests)
        cache.allocate(self.rt.device, self.rt.dtype)
        runner = Runner(self.model, cache, self.rt, self.config.max_position_embeddings)
        if graphs:
            runner.enable_graphs((1, 2, 4))          # single-token steps replay captured CUDA graphs
        return runner


@pytest.fixture(scope="module", params=[(n, d) for n in "ABCD" for d in DTYPES], ids=lambda p: f"{p[0]}-{p[1]}")
def case(request, tmp_path_factory):
    return Case(tmp_path_factory.mktemp("models"), *request.param)


def test_each_request_alone_and_whole(case):
    runner = case.runner(num_pages=-(-max(LENGTHS[case.name].values()) // case.page))
    for rid, toks in case.tokens.items():
        close(run_whole(runner, rid, toks), case.want[rid], case.dtype, f"whole {rid}")
    runner.cache.check()


@pytest.mark.parametrize("graphs", [False, True], ids=["eager", "graphs"])
def test_most_in_one_step_then_the_last_32_one_by_one(case, graphs):
    runner = case.runner(num_pages=-(-max(LENGTHS[case.name].values()) // case.page), graphs=graphs)
    for rid, toks in case.tokens.items():
        n = len(toks)
        tail = min(32, n - 1)
        sizes = ([n - tail] if n - tail else []) + [1] * tail
        close(run_portions(runner, rid, toks, sizes), case.want[rid], case.dtype, f"decode tail {rid}")


def test_portions_of_changing_size(case):
    runner = case.runner(num_pages=-(-max(LENGTHS[case.name].values()) // case.page))
    for k, (rid, toks) in enumerate(case.tokens.items()):
        cycle = [[7, 2, 13, 3, 2, 5], [2, 2, 31, 2, 17], [64, 2, 3]][k % 3]
        close(run_portions(runner, rid, toks, portions(len(toks), cycle)), case.want[rid], case.dtype, f"portions {rid}")


@pytest.mark.parametrize("graphs", [False, True], ids=["eager", "graphs"])
def test_mixed_batches_with_pages_used_again(case, graphs):
    rng = random.Random(7)
    lengths = LENGTHS[case.name]
    need = sorted((-(-n // case.page) for n in lengths.values()), reverse=True)
    runner = case.runner(num_pages=sum(need[:4]), graphs=graphs)        # four live requests fit only through reuse
    steps = mixed_schedule(rng, lengths, max_live=4, decode_tail=9)
    assert any(len(e) >= 3 and any(n == 1 for _, n in e) and any(n > 1 for _, n in e) for e, _ in steps)
    got = run_mixed(runner, case.tokens, steps)
    for rid in case.tokens:
        close(got[rid], case.want[rid], case.dtype, f"mixed {rid}")
    runner.cache.check()
    assert all(g.pool.num_held == 0 for g in runner.cache.groups)
    # and once more over the same pool, in another order: every page has been used before
    steps = mixed_schedule(random.Random(8), dict(reversed(list(lengths.items()))), max_live=3, decode_tail=4)
    got = run_mixed(runner, case.tokens, steps)
    for rid in case.tokens:
        close(got[rid], case.want[rid], case.dtype, f"mixed again {rid}")


def test_long_decoding(case):
    """A short prompt, then every further token one by one up to the context limit."""
    n = case.raw["max_position_embeddings"]
    toks = random_prompt(random.Random(9), case.raw["vocab_size"], n)
    want = plain_forward(case.cfg, case.w, toks, case.dtype)
    runner = case.runner(num_pages=-(-n // case.page), graphs=True)
    runner.GRAPH_MIN_SPAN = 32           # several graphs on the way: one per span of lengths (32, 64, 128, ...)
    close(run_portions(runner, "long", toks, [5] + [1] * (n - 5)), want, case.dtype, "long decoding")
    assert len(runner.graphs) >= 3


def test_first_tokens_of_a_sequence(case):
    runner = case.runner(num_pages=8)
    rng = random.Random(10)
    for n in (1, 2, 3, 5):
        toks = random_prompt(rng, case.raw["vocab_size"], n)
        want = plain_forward(case.cfg, case.w, toks, case.dtype)
        close(run_whole(runner, f"w{n}", toks), want, case.dtype, f"first {n} whole")
        close(run_portions(runner, f"p{n}", toks, [1] * n), want, case.dtype, f"first {n} one by one")


def test_greedy_generation_through_the_entry_point(case):
    from marin_b200 import Engine, SamplingParams, StopReason

    engine = Engine(case.dir, dtype=case.dtype, ctx=case.raw["max_position_embeddings"], page_size=case.page,
                    max_batch=3, token_budget=24)
    rng = random.Random(12)
    prompts = [random_prompt(rng, case.raw["vocab_size"], n) for n in (5, 30, 1, 12)]
    outs = engine.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12))
    assert [o.stop for o in outs] == [StopReason.MAX_TOKENS] * 4
    for prompt, out in zip(prompts, outs):
        assert len(out.tokens) == 12
        if case.dtype == "float32":
            assert out.tokens == plain.greedy(case.cfg, case.w, prompt, 12)
        else:
            # bfloat16 may pick another token where two logits are nearly equal: every token must be
            # (nearly) the best one given the tokens before it
            ids = list(prompt)
            for tok in out.tokens:
                row = plain.forward(case.cfg, case.w, ids)[-1]
                assert float(row.max() - row[tok]) <= 0.15
                ids.append(tok)
    engine.cache.check()
    assert not engine.cache.requests


def test_steps_packed_or_launched_ahead_change_nothing(case):
    """While a decode step runs the engine supposes that the same requests go on: it packs the next step's inputs, and
    where everybody decodes greedily it even launches that step, fed with the token ids the running step leaves on the
    device, before the host has seen them.  The supposition fails when a request ends on a stop token, is cancelled or
    another joins: requests of different lengths, one that stops on a token it is known to produce, one added and one
    cancelled half way, run with steps launched ahead, with steps only packed ahead, and with neither, must give the
    same tokens; and the steps launched or packed ahead must really have been used."""
    from marin_b200 import Engine, SamplingParams

    rng = random.Random(31)
    prompts = [random_prompt(rng, case.raw["vocab_size"], n) for n in (9, 3, 17, 6)]

    def run(pack: bool, launch: bool):
        engine = Engine(case.dir, dtype=case.dtype, ctx=case.raw["max_position_embeddings"], page_size=case.page,
                        max_batch=4, token_budget=32)
        engine.prepare_ahead, engine.run_ahead = pack, launch
        used = {"packed": 0, "launched": 0}
        packed, launched = engine.runner._run_prepared, engine.runner.launch_ahead
        engine.runner._run_prepared = lambda *a: (used.__setitem__("packed", used["packed"] + 1), packed(*a))[1]

        def count_launch(entries):
            handle = launched(entries)
            used["launched"] += handle is not None
            return handle
        engine.runner.launch_ahead = count_launch
        first = engine.generate([prompts[0]], SamplingParams(temperature=0.0, max_tokens=10))[0].tokens
        stop = first[6]                                       # request 0 run again ends when it produces this token
        ids = [engine.add_request(prompts[0], SamplingParams(temperature=0.0, max_tokens=30, stop_tokens=(stop,))),
               engine.add_request(prompts[1], SamplingParams(temperature=0.0, max_tokens=14)),
               engine.add_request(prompts[2], SamplingParams(temperature=0.0, max_tokens=25))]
        out = {i: [] for i in ids}
        steps = 0
        while engine.scheduler.has_work():
            for rid, tok in engine.step():
                out[rid].append(tok)
            steps += 1
            if steps == 8:
                late = engine.add_request(prompts[3], SamplingParams(temperature=0.0, max_tokens=9))
                ids.append(late)
                out[late] = []
            if steps == 16:
                engine.scheduler.cancel(ids[2])
            assert steps < 200
        for i in ids:
            engine.forget(i)
        engine.cache.check()
        assert not engine.cache.requests
        assert [engine.generate([prompts[0]], SamplingParams(temperature=0.0, max_tokens=10))[0].tokens] == [first]   # and once more after all that
        engine.cache.check()
        assert not engine.cache.requests and all(g.pool.num_held == 0 for g in engine.cache.groups)
        return first, [out[i] for i in ids], used

    first_a, launched_ahead, used_a = run(True, True)
    first_b, packed_ahead, used_b = run(True, False)
    first_c, neither, used_c = run(False, False)
    assert used_a["launched"] >= 10 and used_b["packed"] >= 10 and used_b["launched"] == 0 and used_c == {"packed": 0, "launched": 0}
    assert first_a == first_b == first_c and launched_ahead == packed_ahead == neither
    assert len(neither[0]) == first_a.index(first_a[6])   # the stop token itself is not emitted
    assert len(neither[1]) == 14 and len(neither[3]) == 9


def test_a_wait_that_gave_up_is_reported(case):
    """Kernels bound their waits and leave a code on the device when one gives up; the sampling kernel that ends a step
    copies it beside the sampled ids, so the engine learns of it with the very step it happened in and raises.  The
    code is planted here (nothing on the GPU is made to fail)."""
    if case.name not in "AD" or case.dtype != "bfloat16":
        pytest.skip("two configurations are enough")
    from marin_b200 import Engine, SamplingParams
    from marin_b200.kernels.ops import KernelError

    engine = Engine(case.dir, dtype=case.dtype, ctx=case.raw["max_position_embeddings"], page_size=case.page, max_batch=2, token_budget=16)
    engine.generate([[1, 2, 3]], SamplingParams(temperature=0.0, max_tokens=3))
    flag = engine.runner.scratch.error
    flag.fill_(13)
    with pytest.raises(KernelError, match="13"):
        engine.generate([[1, 2, 3]], SamplingParams(temperature=0.0, max_tokens=3))
    assert int(flag.item()) == 0 and int(engine.runner.scratch.report[0].item()) == 0      # read and cleared
    engine.cache.check()
    assert not engine.cache.requests                          # the failed generation left nothing behind
    # the add_request / step way: the step after the flag is raised sees it, whether it samples eagerly or from a graph
    engine.add_request([4, 5, 6], SamplingParams(temperature=0.0, max_tokens=8))
    engine.step()
    engine.step()
    flag.fill_(14)
    with pytest.raises(KernelError, match="14"):
        engine.step()                                         # the step that ran ahead was launched before the flag went up ...
        engine.step()                                         # ... so the one after it brings the news
    engine.check_device()                                     # nothing is left to report


def test_schedule_may_repeat_a_layer_and_share_a_cache(case):
    """The order layers run in is data: layer 0 twice, the second run reading the first run's cache."""
    if case.name != "A":
        pytest.skip("one configuration is enough")
    from marin_b200.cache import CacheManager
    from marin_b200.engine import Runner, build_model
    from marin_b200.models import architecture_of
    from marin_b200.parts import ScheduleEntry
    from marin_b200.models.model import Model
    from marin_b200.weights import load_tensors

    spec = architecture_of(case.config).build_spec(case.config)
    spec.schedule = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(1), ScheduleEntry(0, cache_of=0)]
    model = Model(spec)
    model.load(load_tensors(case.dir, model.tensor_specs(), spec.ignorable), case.rt)
    cache = CacheManager(model.cache_needs(), [e.cache_of for e in spec.schedule], case.page, 40, 4)
    cache.allocate(case.rt.device, case.rt.dtype)
    assert len(cache.groups) == 1 and len(cache.groups[0].entries) == 3
    runner = Runner(model, cache, case.rt, 128)
    toks = case.tokens["a"]
    want = plain_forward(case.cfg, case.w, toks, case.dtype, schedule=[(0, None), (1, None), (1, None), (0, 0)])
    close(run_whole(runner, "w", toks), want, case.dtype, "schedule whole")
    close(run_portions(runner, "p", toks, portions(len(toks), [5, 2, 1, 9])), want, case.dtype, "schedule portions")
