"""The scheduler's decisions (with a fake step: no model) and the sampler."""
import random

import numpy as np
import pytest

from marin_b200.cache import CacheManager
from marin_b200.engine import Request, RequestError, Scheduler, StopReason
from marin_b200.parts import PagedKV
from marin_b200.sampling import Sampler, SamplerError, SamplingParams, best_index


def sched(num_pages=16, page=4, max_batch=3, budget=8, ctx=32):
    cache = CacheManager([PagedKV(1, 8, None)], [None], page, num_pages, max_batch)
    return Scheduler(cache, max_batch, budget, ctx), cache


def reserve_ahead(cache, plan, ctx) -> bool:
    """What the engine does while a decode step runs: the same requests' next token gets its pages now, all or none."""
    import ctypes

    n = len(plan)
    handles = np.fromiter((cache.requests[p.request.req_id].handle for p in plan), np.int64, n)
    counts = np.ones(n, np.int32)
    info = (ctypes.c_int * 2)()
    return cache._lib.mbh_step_reserve(cache._core(), n, handles.ctypes.data, counts.ctypes.data, ctx, info) == 0


def run(s, cache, next_token=lambda r: len(r.tokens) % 50 + 1, max_steps=500, ahead_ctx=0):
    """Drives the scheduler with a fake step that only does the cache bookkeeping.  ``ahead_ctx`` > 0: after every
    step in which all requests decode, pages for their next tokens are taken ahead (context capacity ``ahead_ctx``)."""
    log = []
    for _ in range(max_steps):
        if not s.has_work():
            break
        plan = s.schedule()
        if not plan:
            continue
        for p in plan:
            new_len = p.request.computed + len(p.tokens)
            cache.reserve(p.request.req_id, new_len)
            cache.commit(p.request.req_id, new_len)
        cache.check()
        log.append([(p.request.req_id, len(p.tokens), p.sample) for p in plan])
        if ahead_ctx and all(p.sample and len(p.tokens) == 1 for p in plan):
            reserve_ahead(cache, plan, ahead_ctx)
            cache.check()
        s.update(plan, {p.request.req_id: next_token(p.request) for p in plan if p.sample})
    assert not s.has_work()
    return log


def greedy(max_tokens, stop=()):
    return SamplingParams(temperature=0.0, max_tokens=max_tokens, stop_tokens=tuple(stop))


def test_prompts_are_cut_under_the_token_budget_and_decodes_go_first():
    s, cache = sched(budget=8)
    s.add(Request("a", list(range(1, 14)), greedy(3)))
    s.add(Request("b", list(range(1, 6)), greedy(2)))
    log = run(s, cache)
    assert log[0] == [("a", 8, False)]                              # a portion, no sampling yet
    assert log[1] == [("a", 5, True), ("b", 3, False)]              # the rest of a, then b gets what is left
    assert log[2] == [("a", 1, True), ("b", 2, True)]               # a decodes beside b's last portion
    assert log[3] == [("a", 1, True), ("b", 1, True)]
    assert all(n <= 8 for step in log for n in [sum(e[1] for e in step)])
    done = {r.req_id: r for r in s.finished}
    assert done["a"].stop == StopReason.MAX_TOKENS and len(done["a"].output) == 3 and len(done["b"].output) == 2
    assert cache.free_pages() == [16] and not cache.requests


def test_max_batch_limits_admission_and_finishing_frees():
    s, cache = sched(max_batch=2, budget=16)
    for rid in "abc":
        s.add(Request(rid, [1, 2, 3], greedy(2)))
    log = run(s, cache)
    assert [e[0] for e in log[0]] == ["a", "b"]                     # c waits for a slot
    assert any(e[0] == "c" for e in log[2])                         # admitted when a and b are done
    assert all(len(step) <= 2 for step in log)


def test_stop_token_is_not_emitted_and_max_tokens_zero_does_nothing():
    s, cache = sched()
    s.add(Request("a", [1, 2, 3], greedy(10, stop=[6])))
    s.add(Request("z", [1, 2, 3], greedy(0)))
    log = run(s, cache, next_token=lambda r: len(r.tokens) + 1)     # 4, 5, 6 -> stop at 6
    a = next(r for r in s.finished if r.req_id == "a")
    z = next(r for r in s.finished if r.req_id == "z")
    assert a.output == [4, 5] and a.stop == StopReason.END_OF_TEXT
    assert z.output == [] and z.stop == StopReason.MAX_TOKENS and all(e[0] != "z" for step in log for e in step)


def test_empty_and_oversized_prompts_are_refused_and_context_full_ends_a_request():
    s, cache = sched(ctx=8, budget=8)
    with pytest.raises(RequestError, match="empty"):
        s.add(Request("e", [], greedy(1)))
    with pytest.raises(RequestError, match="context"):
        s.add(Request("l", list(range(9)), greedy(1)))
    s.add(Request("a", [1, 2, 3, 4, 5, 6], greedy(10)))
    run(s, cache)
    a = s.finished[-1]
    assert a.stop == StopReason.CONTEXT_FULL and len(a.prompt) + len(a.output) == 9 and a.computed == 8


def test_when_pages_run_out_the_newest_request_is_preempted_and_recomputed():
    # 6 pages of 4: two requests of 8 prompt tokens fill 4 pages; decoding needs a third page each
    s, cache = sched(num_pages=6, budget=16, max_batch=2)
    s.add(Request("old", list(range(1, 9)), greedy(12)))
    s.add(Request("new", list(range(1, 9)), greedy(12)))
    log = run(s, cache)
    done = {r.req_id: r for r in s.finished}
    assert done["old"].preemptions == 0 and done["new"].preemptions >= 1
    assert done["old"].stop == done["new"].stop == StopReason.MAX_TOKENS
    assert len(done["old"].output) == len(done["new"].output) == 12
    # after the preemption `new` comes back with its prompt and what it had generated, as one portion
    back = [e for step in log for e in step if e[0] == "new" and e[1] > 8]
    assert back and back[0][2]
    assert cache.free_pages() == [6]


def test_a_request_that_cannot_fit_alone_fails_clearly():
    s, cache = sched(num_pages=2, budget=16, ctx=32)
    s.add(Request("big", list(range(1, 13)), greedy(4)))           # 12 tokens need 3 pages, 2 exist
    s.add(Request("grows", [1, 2, 3, 4, 5, 6, 7], greedy(8)))      # fits at first, then outgrows the pool
    run(s, cache)
    done = {r.req_id: r for r in s.finished}
    assert done["big"].stop == StopReason.OUT_OF_PAGES and done["big"].output == []
    assert done["grows"].stop == StopReason.OUT_OF_PAGES and len(done["grows"].output) == 2
    assert cache.free_pages() == [2] and not cache.requests


def test_random_arrivals_finish_everything():
    rng = random.Random(3)
    s, cache = sched(num_pages=10, budget=7, max_batch=3, ctx=32)
    want = {}
    for i in range(12):
        n, m = rng.randint(1, 20), rng.randint(1, 10)
        s.add(Request(i, [rng.randint(1, 40) for _ in range(n)], greedy(m)))
        want[i] = min(m, 32 - n + 1)
    run(s, cache, max_steps=2000)
    assert sorted(r.req_id for r in s.finished) == list(range(12))
    for r in s.finished:
        assert len(r.output) == want[r.req_id], (r.req_id, r.stop)
    assert cache.free_pages() == [10]


@pytest.mark.parametrize("pages", [6, 7, 10, 40])
def test_pages_taken_ahead_for_the_next_decode_step_change_no_outcome(pages):
    """The engine reserves the next decode step's pages while the current one runs.  Whatever the pool (so tight that
    requests are preempted, or roomy), every request ends as it does without that, with the same tokens, and every
    page comes back."""
    outcomes = []
    for ahead in (0, 32):
        rng = random.Random(11)
        s, cache = sched(num_pages=pages, budget=9, max_batch=3, ctx=32)
        for i in range(10):
            n, m = rng.randint(1, 18), rng.randint(1, 12)
            stop = (7,) if i % 3 == 0 else ()
            s.add(Request(i, [rng.randint(1, 40) for _ in range(n)], greedy(m, stop)))
        run(s, cache, next_token=lambda r: (len(r.prompt) * 7 + len(r.output) * 3) % 11 + 1, max_steps=3000, ahead_ctx=ahead)
        assert cache.free_pages() == [pages] and not cache.requests
        outcomes.append(sorted((r.req_id, r.stop, tuple(r.output)) for r in s.finished))
    assert outcomes[0] == outcomes[1]
    assert len(outcomes[0]) == 10


@pytest.mark.parametrize("seed", range(8))
def test_requests_added_and_cancelled_at_random_times_with_and_without_pages_taken_ahead(seed):
    """A random programme of arrivals and cancellations over a tight pool, run twice: the second time pages for the next
    decode step are taken ahead after every all-decode step, as the engine does.  The accounting holds at every step,
    every page comes back, and every request ends the same way with the same tokens."""
    rng = random.Random(100 + seed)
    pages, ctx = rng.choice([5, 8, 12, 30]), 40
    programme = []                                            # (step, "add", id, prompt, max_tokens, stop) / (step, "cancel", id)
    for i in range(14):
        at = rng.randint(0, 40)
        programme.append((at, "add", i, [rng.randint(1, 30) for _ in range(rng.randint(1, 22))], rng.randint(1, 14),
                          (5,) if rng.random() < 0.3 else ()))
        if rng.random() < 0.35:
            programme.append((at + rng.randint(1, 12), "cancel", i))
    outcomes = []
    for ahead in (False, True):
        s, cache = sched(num_pages=pages, page=4, max_batch=3, budget=10, ctx=ctx)
        known = {}
        for step in range(400):
            for ev in programme:
                if ev[0] != step:
                    continue
                if ev[1] == "add":
                    known[ev[2]] = Request(ev[2], ev[3], greedy(ev[4], ev[5]))
                    s.add(known[ev[2]])
                elif ev[2] in known:
                    s.cancel(ev[2])
            if not s.has_work():
                if step > 60:
                    break
                continue
            plan = s.schedule()
            for p in plan:
                new_len = p.request.computed + len(p.tokens)
                cache.reserve(p.request.req_id, new_len)
                cache.commit(p.request.req_id, new_len)
            cache.check()
            if ahead and plan and all(p.sample and len(p.tokens) == 1 for p in plan):
                reserve_ahead(cache, plan, ctx)
                cache.check()
            if plan:
                s.update(plan, {p.request.req_id: (len(p.request.prompt) * 5 + len(p.request.output) * 3 + p.request.req_id) % 9 + 1
                                for p in plan if p.sample})
        assert not s.has_work()
        assert cache.free_pages() == [pages] and not cache.requests
        outcomes.append(sorted((r.req_id, r.stop, tuple(r.output)) for r in s.finished))
    assert outcomes[0] == outcomes[1] and len(outcomes[0]) == 14


# ---- sampler ---------------------------------------------------------------------------------------------

def plain_distribution(logits, temperature, top_k, top_p):
    """The reference's plain algorithm written out (crates/sampler/src/lib.rs:59-62,169-193)."""
    order = sorted(range(len(logits)), key=lambda i: (-logits[i], i))
    if top_k:
        order = order[:top_k]
    top = logits[order[0]]
    w = [np.exp(np.float32((logits[i] - top) / np.float32(temperature))) for i in order]
    total = np.float32(0)
    for x in w:
        total = np.float32(total + x)
    kept, mass = [], np.float32(0)
    for i, x in zip(order, w):
        p = np.float32(x / total)
        kept.append((i, p))
        mass = np.float32(mass + p)
        if mass >= np.float32(top_p):
            break
    km = np.float32(0)
    for _, p in kept:
        km = np.float32(km + p)
    return [(i, float(np.float32(p / km))) for i, p in kept]


def test_greedy_lowest_id_wins_ties_and_signed_zero():
    assert best_index(np.array([1.0, 3.0, 3.0, 2.0], np.float32)) == 1
    assert best_index(np.array([-0.0, 0.0, 0.0], np.float32)) == 1          # +0.0 ranks above -0.0
    s = Sampler(SamplingParams(temperature=0.0))
    assert s.sample(np.array([0.5, 9.0, 9.0, 1.0], np.float32)) == 1
    assert s.sample(np.array([0.5, 9.0, 10.0, 11.0], np.float32), usable=3) == 2


@pytest.mark.parametrize("temperature,top_k,top_p", [(0.7, 0, 0.9), (1.0, 5, 1.0), (0.3, 50, 0.5), (2.0, 0, 1.0), (0.7, 1, 0.9), (1.3, 200, 0.99)])
def test_distribution_equals_the_plain_algorithm(temperature, top_k, top_p):
    rng = np.random.default_rng(4)
    for size in (3, 50, 1000):
        logits = (rng.standard_normal(size) * 3).astype(np.float32)
        logits[size // 2] = logits[0]                                      # a tie
        got = Sampler(SamplingParams(temperature=temperature, top_k=top_k, top_p=top_p)).distribution(logits)
        want = plain_distribution(logits, temperature, top_k, top_p)
        assert [i for i, _ in got] == [i for i, _ in want]
        assert np.allclose([p for _, p in got], [p for _, p in want], rtol=1e-5)
        assert abs(sum(p for _, p in got) - 1.0) < 1e-5


def test_sampling_is_seeded_and_follows_the_distribution():
    logits = np.array([2.0, 1.0, 0.0, -1.0], np.float32)
    p = SamplingParams(temperature=1.0, top_k=0, top_p=1.0, seed=42)
    a, b = Sampler(p), Sampler(p)
    draws = [a.sample(logits) for _ in range(2000)]
    assert draws == [b.sample(logits) for _ in range(2000)]
    assert [Sampler(SamplingParams(temperature=1.0, top_p=1.0, seed=43)).sample(logits) for _ in range(20)] != draws[:20]
    freq = np.bincount(draws, minlength=4) / 2000
    want = np.exp(logits) / np.exp(logits).sum()
    assert np.abs(freq - want).max() < 0.04
    # splitmix64 first outputs for seed 0 (public test vector of the generator): top 24 bits of 0xE220A8397B1DCDAF
    s = Sampler(SamplingParams(temperature=1.0, seed=0))
    assert s.next_unit() == (0xE220A8397B1DCDAF >> 40) / 16777216.0


def test_sampler_errors():
    with pytest.raises(SamplerError, match="temperature"):
        Sampler(SamplingParams(temperature=-1.0))
    with pytest.raises(SamplerError, match="top_p"):
        Sampler(SamplingParams(top_p=0.0))
    s = Sampler(SamplingParams(temperature=0.5))
    with pytest.raises(SamplerError, match="NaN"):
        s.sample(np.array([1.0, float("nan")], np.float32))
    with pytest.raises(SamplerError, match="candidates"):
        s.sample(np.array([1.0, 2.0], np.float32), usable=0)


def test_a_negative_token_ends_its_request_as_non_finite_and_the_others_go_on():
    """The sampler answers -1 for a row whose logits were not finite: that request ends, nothing is emitted for it,
    its pages go back, and the requests beside it are untouched."""
    s, cache = sched()
    s.add(Request("a", [1, 2, 3], greedy(6)))
    s.add(Request("b", [4, 5], greedy(4)))
    run(s, cache, next_token=lambda r: -1 if r.req_id == "a" and len(r.output) == 2 else len(r.tokens))
    a = next(r for r in s.finished if r.req_id == "a")
    b = next(r for r in s.finished if r.req_id == "b")
    assert a.stop == StopReason.NON_FINITE_LOGITS and len(a.output) == 2
    assert b.stop == StopReason.MAX_TOKENS and len(b.output) == 4
    cache.check()
    assert all(g.pool.num_held == 0 for g in cache.groups)
