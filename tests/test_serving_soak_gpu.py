"""An engine at Qwen3-4B widths serving requests that arrive in bursts, for a few hundred steps, twice.

What single tests do not reach: every size of decode batch from 1 to 64 in one run (graphs captured as they are first
needed, rows that pad them), prompt portions of every length beside decoding requests, a pool so small that running
requests are preempted and recomputed again and again, all with dependent launches back to back for seconds.  A fault
that needs a rare overlap of neighbouring kernels shows here sooner than anywhere else (the small-batch product once
had one at 17 to 32 tokens).  Checked: no kernel's bounded wait gave up, no page is lost or held at the end, and the
second run, with the same arrivals, produces the same tokens as the first (nothing in a step depends on timing).  The
tokens themselves are held to the plain implementation elsewhere (tests/test_real_widths_gpu.py).

The reference serves its requests one after another (crates/cli/src/server/sched.rs:150-162); it has no counterpart of
this run.
"""
import random

import pytest

pytestmark = pytest.mark.gpu

VOCAB = 8200
LAYERS = 2


def serve(cfg, seed, budget, pages, arrivals_wanted):
    from marin_b200 import Engine, SamplingParams

    engine = Engine(config=cfg, seed=1, dtype="bfloat16", ctx=2048, page_size=16, max_batch=64, token_budget=budget, num_pages=pages)
    rng = random.Random(seed)
    results, pending, steps, arrivals = {}, {}, 0, 0
    while arrivals < arrivals_wanted or engine.has_work():
        if arrivals < arrivals_wanted and (not engine.has_work() or rng.random() < 0.15):
            for _ in range(rng.choice((1, 1, 2, 5, 17, 40))):              # a burst now and then
                if arrivals >= arrivals_wanted:
                    break
                prompt = [rng.randrange(VOCAB) for _ in range(rng.choice((1, 2, 3, 17, 60, 129, 300, 700, 1100)))]
                rid = engine.add_request(prompt, SamplingParams(temperature=0.0, max_tokens=rng.choice((1, 3, 9, 33, 70))))
                pending[rid] = arrivals
                arrivals += 1
        engine.step()
        steps += 1
        for rid in list(pending):
            res = engine.result(rid)
            if res.stop is not None:
                results[pending.pop(rid)] = (tuple(res.tokens), res.stop, res.preemptions)
                engine.forget(rid)
        assert steps < 50 * arrivals_wanted, "the engine makes no progress"
    engine.check_device()
    engine.cache.check()
    assert not engine.cache.requests and all(g.pool.num_held == 0 for g in engine.cache.groups)
    return results, steps, sorted(b for (b, _span) in engine.runner.graphs)


@pytest.mark.parametrize("budget,pages", [(512, 250), (2048, 3000)])
def test_bursts_of_requests_for_hundreds_of_steps_twice(budget, pages):
    from marin_b200.config import Qwen3Config
    from test_real_widths_gpu import LAYOUTS

    cfg = Qwen3Config.from_dict(dict(LAYOUTS["4b"], num_hidden_layers=LAYERS))
    first, steps, buckets = serve(cfg, 7, budget, pages, 500)
    second, _, _ = serve(cfg, 7, budget, pages, 500)
    assert len(first) == 500 and steps > 300
    if pages < 1000:
        assert sum(v[2] for v in first.values()) > 10                     # the small pool preempted again and again
        assert len(set(buckets)) >= 4
    else:
        assert len(set(buckets) & {1, 2, 4, 8, 16, 32, 64}) >= 6          # (nearly) every size of captured batch ran
    differ = [k for k in first if first[k] != second.get(k)]
    assert not differ, f"requests {differ[:8]} got other tokens in the second run"
