"""Schedules of the entry point that the other engine tests do not reach, on the GPU against the plain implementation:
a pool so small that a running request is preempted and recomputed; the host sampler inside the engine beside the
device sampler on one seeded batch of greedy and sampled requests; logits that must not depend on the cut by a single
bit (float32) nor differ between two runs of one schedule (both dtypes); and a request whose logits are not finite.

What the reference does where this engine preempts: a starved request waits for another to finish
(crates/cli/src/server/sched.rs:150-162).  Its chunking gate: crates/model/tests/kv_append.rs:84-148.
"""
import random

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from helpers import mixed_schedule, portions, random_prompt, run_mixed, run_portions, run_whole
from test_engine_gpu import LENGTHS, Case, close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", params=[(n, d) for n in "ABD" for d in ("float32", "bfloat16")], ids=lambda p: f"{p[0]}-{p[1]}")
def case(request, tmp_path_factory):
    return Case(tmp_path_factory.mktemp("models"), *request.param)


def near_best(case, prompt, tokens, margin=0.15):
    """Every token is (nearly) the best one given the tokens before it, by the plain implementation."""
    ids = list(prompt)
    for tok in tokens:
        row = plain.forward(case.cfg, case.w, ids)[-1]
        assert float(row.max() - row[tok]) <= margin
        ids.append(tok)


def test_a_request_preempted_for_want_of_pages_is_recomputed_and_emits_the_same_tokens(case):
    from marin_b200 import Engine, SamplingParams, StopReason

    page, limit = case.page, case.raw["max_position_embeddings"]
    rng = random.Random(41)
    new = 40
    prompts = [random_prompt(rng, case.raw["vocab_size"], n) for n in (20, 25, 30)]
    at_start = sum(-(-len(p) // page) for p in prompts)
    at_end = sum(-(-(len(p) + new) // page) for p in prompts)
    pool = at_start + (at_end - at_start) // 2 + 1          # all three start; they cannot all finish side by side
    assert -(-(30 + new) // page) <= pool < at_end
    engine = Engine(case.dir, dtype=case.dtype, ctx=limit, page_size=page, num_pages=pool, max_batch=3, token_budget=64)
    outs = engine.generate(prompts, SamplingParams(temperature=0.0, max_tokens=new))
    assert [o.stop for o in outs] == [StopReason.MAX_TOKENS] * 3
    assert sum(o.preemptions for o in outs) >= 1            # the newest running request gave its pages back at least once
    for prompt, out in zip(prompts, outs):
        assert len(out.tokens) == new
        if case.dtype == "float32":
            assert out.tokens == plain.greedy(case.cfg, case.w, prompt, new)
        else:
            near_best(case, prompt, out.tokens)
    engine.cache.check()
    assert not engine.cache.requests and all(g.pool.num_held == 0 for g in engine.cache.groups)
    # the same prompts with room for everything: nobody is preempted, and in float32 the tokens are the same ones
    roomy = Engine(case.dir, dtype=case.dtype, ctx=limit, page_size=page, max_batch=3, token_budget=64)
    again = roomy.generate(prompts, SamplingParams(temperature=0.0, max_tokens=new))
    assert sum(o.preemptions for o in again) == 0
    if case.dtype == "float32":
        assert [o.tokens for o in again] == [o.tokens for o in outs]


def test_host_sampler_and_device_sampler_in_one_seeded_batch(case):
    """Greedy requests beside sampled ones in the same steps.  With ``device_sampling=False`` every token comes from
    the host sampler (the reference's algorithm): in float32 that must be the token the host sampler draws from the
    plain implementation's logits with the same seed.  The device sampler draws from the same kept set (temperature,
    top-k, top-p) but walks it in id order, so a sampled request may take another member of the set; greedy requests
    must get the same tokens either way."""
    from marin_b200 import Engine, Sampler, SamplingParams

    if case.name == "D":
        pytest.skip("two configurations are enough")
    rng = random.Random(43)
    vocab = case.raw["vocab_size"]
    prompts = [random_prompt(rng, vocab, n) for n in (7, 19, 3, 12)]
    params = [SamplingParams(temperature=0.0, max_tokens=10),
              SamplingParams(temperature=0.8, top_k=12, top_p=0.9, seed=5, max_tokens=10),
              SamplingParams(temperature=1.3, top_k=0, top_p=0.6, seed=6, max_tokens=10),
              SamplingParams(temperature=0.0, max_tokens=10)]

    def run(device_sampling):
        engine = Engine(case.dir, dtype=case.dtype, ctx=case.raw["max_position_embeddings"], page_size=case.page, max_batch=4,
                        token_budget=32, device_sampling=device_sampling)
        return [o.tokens for o in engine.generate(prompts, params)]

    host, device = run(False), run(True)
    assert host[0] == device[0] and host[3] == device[3]                     # the greedy rows
    if case.dtype == "float32":
        assert host[0] == plain.greedy(case.cfg, case.w, prompts[0], 10)
        for i in (1, 2):
            # the host path: the very tokens the host sampler draws from the plain logits, seed and all
            sampler, ids = Sampler(params[i]), list(prompts[i])
            for tok in host[i]:
                row = plain.forward(case.cfg, case.w, ids)[-1].numpy()
                assert tok == sampler.sample(row), f"request {i}: the engine's host sampler and a host sampler fed plain logits disagree"
                ids.append(tok)
            # the device path: every token lies in the set the host sampler keeps for the tokens before it
            ids = list(prompts[i])
            for tok in device[i]:
                row = plain.forward(case.cfg, case.w, ids)[-1].numpy()
                kept = [t for t, _ in Sampler(params[i]).distribution(row)]
                assert tok in kept, f"request {i}: token {tok} is outside the kept set of {len(kept)}"
                ids.append(tok)
    else:
        for i in (1, 2):
            assert len(host[i]) == 10 and len(device[i]) == 10 and all(0 <= t < vocab for t in host[i] + device[i])


def test_float32_logits_do_not_depend_on_the_cut_by_a_single_bit(case):
    """The float32 path sums every output value in one fixed order whatever else is in the batch, so whole, tail,
    portions and mixed runs of one request must agree in every bit, not merely within the tolerance.  In bfloat16 the
    split of K and of the keys follows the batch, so the cuts differ by rounding; but the same schedule run twice
    must give the same bits in both dtypes: nothing in a step depends on timing."""
    lengths = LENGTHS[case.name]
    rid = max(lengths, key=lengths.get)
    toks = case.tokens[rid]
    n = len(toks)
    need = sorted((-(-m // case.page) for m in lengths.values()), reverse=True)

    def mixed(seed):
        runner = case.runner(num_pages=sum(need[:4]), graphs=True)
        return run_mixed(runner, case.tokens, mixed_schedule(random.Random(seed), lengths, max_live=4, decode_tail=9))

    first, second = mixed(7), mixed(7)
    for r in lengths:
        assert torch.equal(first[r], second[r]), f"request {r}: two runs of one schedule differ"
    if case.dtype != "float32":
        return
    runner = case.runner(num_pages=-(-n // case.page), graphs=True)
    whole = run_whole(runner, "w", toks)
    tail = run_portions(runner, "t", toks, [n - 32] + [1] * 32)
    cut = run_portions(runner, "p", toks, portions(n, [7, 2, 13, 3, 2, 5]))
    other = mixed(8)
    for what, got in (("tail", tail), ("portions", cut), ("mixed", first[rid]), ("mixed in another order", other[rid])):
        same = (got == whole).all(dim=1)
        assert bool(same.all()), f"{what}: first position whose logits differ from the whole run's: {int(torch.nonzero(~same)[0])} of {n}"


def test_logits_that_are_not_finite_end_their_request_and_no_other(case, tmp_path):
    """A checkpoint in which one embedding row is infinite: every request that holds that token gets NaN logits, is
    ended with NON_FINITE_LOGITS by the step that would have sampled from them, and the error names it; requests beside
    it in the same steps go on and produce the plain implementation's tokens."""
    import json
    import os

    from safetensors.torch import load_file

    from marin_b200 import Engine, SamplingParams, StopReason
    from marin_b200.engine.engine import GenerationError
    from marin_b200.weights import write_safetensors

    if case.name != "B":
        pytest.skip("the untied configuration: the bad row must not be a row of the head")
    bad_token = 7
    d = str(tmp_path / "inf")
    os.makedirs(d)
    tensors = load_file(os.path.join(case.dir, "model.safetensors"))
    table = tensors["model.embed_tokens.weight"].clone()
    table[bad_token, 3] = float("inf")
    tensors["model.embed_tokens.weight"] = table
    write_safetensors(os.path.join(d, "model.safetensors"), tensors.items())
    with open(os.path.join(d, "config.json"), "w") as fh:
        json.dump(case.raw, fh)
    rng = random.Random(47)
    vocab = case.raw["vocab_size"]
    clean = [t for t in random_prompt(rng, vocab, 40) if t != bad_token]
    good_a, good_b = clean[:11], clean[11:30]
    poisoned = clean[30:36] + [bad_token] + clean[36:39]
    for device_sampling in (True, False):
        engine = Engine(d, dtype=case.dtype, ctx=128, page_size=case.page, max_batch=3, token_budget=64, device_sampling=device_sampling)
        ids = [engine.add_request(p, SamplingParams(temperature=0.0, max_tokens=8, stop_tokens=(bad_token,))) for p in (good_a, poisoned, good_b)]
        errors = []
        while engine.has_work():
            try:
                engine.step()
            except GenerationError as err:
                errors.append(err)
        assert len(errors) == 1 and errors[0].req_id == ids[1] and "not finite" in str(errors[0])
        results = [engine.result(i) for i in ids]
        assert results[1].stop == StopReason.NON_FINITE_LOGITS and results[1].tokens == []
        for res, prompt in ((results[0], good_a), (results[2], good_b)):
            assert res.stop in (StopReason.MAX_TOKENS, StopReason.END_OF_TEXT)
            if case.dtype == "float32":
                want = plain.greedy(case.cfg, case.w, prompt, 8)
                want = want[:want.index(bad_token)] if bad_token in want else want
                assert res.tokens == want
            else:
                near_best(case, prompt, res.tokens)
        engine.cache.check()
        assert not engine.cache.requests
        # generate() fails as a whole and leaves nothing behind
        with pytest.raises(GenerationError):
            engine.generate([good_a, poisoned], SamplingParams(temperature=0.0, max_tokens=4, stop_tokens=(bad_token,)))
        engine.cache.check()
        assert not engine.cache.requests and not engine.has_work()
        out = engine.generate([good_a], SamplingParams(temperature=0.0, max_tokens=4, stop_tokens=(bad_token,)))
        assert len(out[0].tokens) <= 4 and out[0].stop in (StopReason.MAX_TOKENS, StopReason.END_OF_TEXT)      # and the engine still serves
