#!/usr/bin/env python3
"""Logit equality at full layer sizes: the engine against the plain implementation at the layer sizes of a real
model (Qwen3-4B, 8B or 14B: every width as in the model, fewer layers so that the plain implementation, on the CPU,
ends in a minute) and a context of 4,096, under every way of cutting the work:

  whole      the prompt in one step;
  tail       all but the last 32 tokens in one step, the last 32 one by one (graphs);
  portions   in portions of changing size, down to two tokens;
  mixed      five requests, three live at a time, portions of some beside decoded tokens of others, in a pool so
             small that pages are used again.

    python tests/check_layout_equality.py [--model 4b|8b|14b] [--layers 2] [--context 4096] [--dtypes float32,bfloat16]

float32 must agree within 1e-4 + 1e-4 |x| at every position, bfloat16 within the tolerances of the tests
(tests/test_engine_gpu.py: close, against the plain result rounded where a 16-bit engine stores).  Too slow for the
test suite (a minute or two of CPU per model); the suite holds the same comparisons on one layer of the same widths
with a cut vocabulary and a context of 1,100 (tests/test_real_widths_gpu.py).  Prints one line per comparison and
exits non-zero if any fails.
"""
import argparse
import math
import os
import random
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="4b", choices=["4b", "8b", "14b"])
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--dtypes", default="float32,bfloat16")
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args()

    import torch

    import bench
    import plain_qwen3 as plain
    from helpers import make_model_dir, mixed_schedule, portions, random_prompt, run_mixed, run_portions, run_whole
    from test_engine_gpu import close, plain_forward

    from marin_b200.cache import CacheManager
    from marin_b200.engine import Runner, load_model, parse_dtype
    from marin_b200.kernels import ops
    from marin_b200.parts import Runtime

    raw = dict(bench.LAYOUTS[args.model])
    raw["num_hidden_layers"] = args.layers
    raw["max_position_embeddings"] = max(args.context, raw.get("max_position_embeddings", args.context))
    n, page, vocab = args.context, bench.PAGE, raw["vocab_size"]
    rng = random.Random(args.seed + 1)
    failures = 0
    with tempfile.TemporaryDirectory() as tmp:
        t0 = time.time()
        # written once, in bfloat16: the float32 run reads the same values, so one plain result serves both
        # matrices of standard deviation 1 / sqrt(width), so that logits have a standard deviation near 1 at every
        # layout (the bfloat16 tolerance is absolute and supposes that)
        folder = make_model_dir(os.path.join(tmp, "m"), raw, seed=args.seed, dtype=torch.bfloat16,
                                matrix_std=1.0 / math.sqrt(raw["hidden_size"]))
        cfg, w = plain.read_config(folder), plain.read_weights(folder)
        print(f"[{time.time() - t0:6.1f} s] {args.model} layout, {args.layers} layers: weights written and read", flush=True)
        prompt = random_prompt(rng, vocab, n)
        lengths = {"a": n, "b": 1000, "c": 300, "d": 2000, "e": 600}
        others = {rid: random_prompt(rng, vocab, min(L, n)) for rid, L in lengths.items() if rid != "a"}
        others["a"] = prompt
        for dtype in args.dtypes.split(","):
            # bfloat16 is held to the plain result rounded where a 16-bit engine stores its activations
            want = {rid: plain_forward(cfg, w, toks, dtype) for rid, toks in others.items()}
            print(f"[{time.time() - t0:6.1f} s] plain implementation for {dtype} done (logits of standard deviation {float(want['a'].std()):.2f})", flush=True)
            rt = Runtime(torch.device("cuda:0"), parse_dtype(dtype))
            _, model = load_model(folder, rt)
            per_seq = -(-n // page)

            def runner_with(pages: int, graphs: bool):
                cache = CacheManager(model.cache_needs(), [e.cache_of for e in model.spec.schedule], page, pages, 4)
                cache.allocate(rt.device, rt.dtype)
                runner = Runner(model, cache, rt, n)
                if graphs:
                    runner.enable_graphs((1, 2, 4))
                return runner

            def check(what: str, got, wanted) -> None:
                nonlocal failures
                try:
                    close(got, wanted, dtype, what)
                    err = float((got.float().cpu() - wanted).abs().max())
                    print(f"[{time.time() - t0:6.1f} s] {dtype:8s} {what:28s} ok   (largest difference {err:.2e})", flush=True)
                except AssertionError as e:
                    failures += 1
                    print(f"[{time.time() - t0:6.1f} s] {dtype:8s} {what:28s} FAIL {e}", flush=True)

            runner = runner_with(per_seq + 2, graphs=True)
            check("whole", run_whole(runner, "w", prompt), want["a"])
            check("tail of 32 decoded", run_portions(runner, "t", prompt, [n - 32] + [1] * 32), want["a"])
            check("portions", run_portions(runner, "p", prompt, portions(n, [512, 2, 1000, 3, 2, 257, 64])), want["a"])
            runner.cache.check()
            need = sorted((-(-len(t) // page) for t in others.values()), reverse=True)
            runner = runner_with(sum(need[:3]) + 1, graphs=True)
            steps = mixed_schedule(random.Random(args.seed + 2), {rid: len(t) for rid, t in others.items()}, max_live=3,
                                   decode_tail=9, sizes=(700, 2, 1300, 3, 2, 500))
            got = run_mixed(runner, others, steps)
            for rid in sorted(others):
                check(f"mixed, request {rid} ({len(others[rid])})", got[rid], want[rid])
            runner.cache.check()
            ops.check_device_errors()
            del runner, model, got
            torch.cuda.empty_cache()
    print("all equal" if failures == 0 else f"{failures} comparison(s) failed")
    return 0 if failures == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
