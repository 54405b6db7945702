"""Command line in the manner of the reference's ``marin-run`` (crates/cli/src/args.rs:41-389).

    marin-run MODEL_DIR -p TEXT | --prompt-ids 1,2,3 [--ctx N] [--max-tokens 128] [--temp 0.7] [--top-k 0]
                        [--top-p 0.9] [--seed N] [--metrics] [--dtype bfloat16|float32]
    marin-run bench MODEL_DIR [--prompt-tokens 128] [--tokens 64] [--runs 3] [--warmup 1] [--temp 0] [--json FILE] [--profile]
    marin-run verify MODEL_DIR --reference REF.json
    marin-run random --config CONFIG.json --seed S --out DIR [--dtype bfloat16|float32]

Option names and defaults are the reference's where it has them (``--temp``, ``--top-k``, ``--top-p``, ``--seed``,
``--max-tokens``, ``--ctx``, ``--prompt-tokens``, ``--tokens``, ``--runs``, ``--warmup``, ``--json``, ``--profile``).  ``-p`` needs
``tokenizer.json`` in the model folder and the ``tokenizers`` package; ``--prompt-ids`` takes token ids and prints
token ids.  The reply goes to stdout, everything else to stderr.  ``random`` (random-weights mode) and ``--dtype``
have no counterpart in the reference; its ``--backend``, ``--quantize``, ``--kv-type``, ``--speculate`` are not taken.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time
from typing import List, Optional

DEFAULT_MAX_TOKENS = 128


def _tokenizer(model_dir: str):
    path = os.path.join(model_dir, "tokenizer.json")
    if not os.path.exists(path):
        raise SystemExit(f"{model_dir} has no tokenizer.json: give --prompt-ids instead of -p")
    try:
        from tokenizers import Tokenizer
    except ImportError as err:
        raise SystemExit("the `tokenizers` package is needed for text prompts; give --prompt-ids instead") from err
    return Tokenizer.from_file(path)


def _add_sampling(ap: argparse.ArgumentParser, temp: float, top_p: float) -> None:
    ap.add_argument("--temp", type=float, default=temp, help="randomness: 0 always picks the likeliest token")
    ap.add_argument("--top-k", type=int, default=0, help="only consider the K likeliest tokens (0 = off)")
    ap.add_argument("--top-p", type=float, default=top_p, help="only consider tokens whose probabilities add up to P")
    ap.add_argument("--seed", type=int, default=None, help="random seed (default: time based)")


def _engine(args, max_batch=1, token_budget=2048):
    from .engine import Engine

    return Engine(args.model_dir, dtype=args.dtype, ctx=args.ctx, max_batch=max_batch, token_budget=token_budget)


def cmd_run(args) -> int:
    from .sampling import SamplingParams

    if (args.prompt is None) == (args.prompt_ids is None):
        raise SystemExit("give exactly one of -p/--prompt TEXT and --prompt-ids IDS")
    tok = None
    if args.prompt is not None:
        tok = _tokenizer(args.model_dir)
        ids = tok.encode(args.prompt, add_special_tokens=False).ids
    else:
        ids = [int(t) for t in args.prompt_ids.replace(",", " ").split()]
    if not ids:
        raise SystemExit("the prompt is empty")
    t0 = time.perf_counter()
    engine = _engine(args)
    load_s = time.perf_counter() - t0
    seed = args.seed if args.seed is not None else time.time_ns() & 0xFFFFFFFF
    params = SamplingParams(temperature=args.temp, top_k=args.top_k, top_p=args.top_p, seed=seed, max_tokens=args.max_tokens,
                            stop_tokens=tuple(engine.config.eos_token_ids))
    pieces: List[int] = []
    stamps: List[float] = []

    def on_token(_rid, token):
        stamps.append(time.perf_counter())
        pieces.append(token)
        if tok is None:
            sys.stdout.write(("" if len(pieces) == 1 else " ") + str(token))
        else:
            sys.stdout.write(tok.decode([token]))
        sys.stdout.flush()

    t1 = time.perf_counter()
    out = engine.generate([ids], params, on_token=on_token)[0]
    sys.stdout.write("\n")
    if args.metrics:
        first = stamps[0] - t1 if stamps else 0.0
        decode = (stamps[-1] - stamps[0]) if len(stamps) > 1 else 0.0
        print(f"load {load_s:.2f} s; prompt {len(ids)} tokens, first token after {first * 1e3:.1f} ms "
              f"({len(ids) / first if first else 0:.0f} tok/s); {len(pieces)} tokens generated, "
              f"{(len(pieces) - 1) / decode if decode else 0:.1f} tok/s after the first; stop: {out.stop.value}", file=sys.stderr)
    return 0


def cmd_bench(args) -> int:
    """Prefill and decode speed of one sequence, the reference's definitions (crates/cli/src/bench/mod.rs:219-231):
    prefill tok/s = prompt tokens / time of the prompt pass; decode tok/s = (generated - 1) / time after the first."""
    import torch

    from .sampling import SamplingParams

    engine = _engine(args, token_budget=max(2048, args.prompt_tokens))
    vocab = engine.config.vocab_size
    g = torch.Generator().manual_seed(args.seed or 0)
    prompt = torch.randint(0, vocab, (args.prompt_tokens,), generator=g).tolist()
    params = SamplingParams(temperature=args.temp, top_k=args.top_k, top_p=args.top_p, seed=args.seed or 0, max_tokens=args.tokens)
    runs = []
    for i in range(args.warmup + args.runs):
        stamps: List[float] = []
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        engine.generate([prompt], params, on_token=lambda _r, _t: stamps.append(time.perf_counter()))
        if i >= args.warmup and stamps:
            first = stamps[0] - t0
            decode = stamps[-1] - stamps[0]
            gaps = [b - a for a, b in zip(stamps, stamps[1:])]
            runs.append({"first_token_ms": first * 1e3, "prefill_tokens_per_s": args.prompt_tokens / first,
                         "decode_tokens_per_s": (len(stamps) - 1) / decode if decode > 0 else 0.0,
                         "gap_p50_ms": statistics.median(gaps) * 1e3 if gaps else 0.0})
    record = {"format": 1, "model_dir": args.model_dir, "dtype": args.dtype, "prompt_tokens": args.prompt_tokens,
              "tokens": args.tokens, "runs": args.runs, "warmup": args.warmup, "batch_size": 1,
              **{k: statistics.median(r[k] for r in runs) for k in runs[0]}}
    print(f"prompt {args.prompt_tokens} tokens: first token {record['first_token_ms']:.1f} ms, prefill "
          f"{record['prefill_tokens_per_s']:.0f} tok/s; decode {record['decode_tokens_per_s']:.1f} tok/s "
          f"(median of {args.runs} runs)")
    if args.json:
        tmp = args.json + ".tmp"
        with open(tmp, "w") as fh:
            json.dump(record, fh, indent=2)
        os.replace(tmp, args.json)
    if args.profile:
        print(profile_text(engine, prompt, args.tokens))
    return 0


def profile_text(engine, prompt: List[int], tokens: int, hbm_gbs: float = 6500.0, peak_tflops: float = 1600.0) -> str:
    """``bench --profile``: where the time of the prompt step and of a decode step goes, stage by stage (the reference's
    flag: crates/cli/src/args.rs:70-91; its stages: crates/metrics/src/stage.rs:5-19).  Fractions are of a B200's
    measured copy bandwidth and library bf16 product rate, about 6.5 TB/s and 1.6 PFLOP/s."""
    from .engine import StepEntry
    from .engine.profile import format_table, profile_steps
    from .kernels import ops

    runner, vocab = engine.runner, engine.config.vocab_size
    out = runner.scratch.ids(1)
    live = []

    def sample(logits):
        ops.stage_name = "sampling"
        ops.argmax(logits, vocab, out)

    def prompt_step(i):
        for rid in live:
            runner.end(rid)
        live[:] = [f"profile{i}"]
        runner.begin(live[0])
        return [StepEntry(live[0], prompt, [len(prompt) - 1])]

    rows = profile_steps(runner, prompt_step, steps=4, warmup=2, after_step=sample)
    text = format_table(rows, hbm_gbs, peak_tflops, f"prompt of {len(prompt)} tokens in one step")
    room = engine.ctx - len(prompt)
    steps = max(1, min(6, room - 3))
    if room >= 2:
        rows = profile_steps(runner, lambda i: [StepEntry(live[0], [prompt[i % len(prompt)]], [0])], steps=steps, warmup=min(3, room - steps),
                             after_step=None if getattr(runner, "graph_sizes", None) else sample)
        text += "\n\n" + format_table(rows, hbm_gbs, peak_tflops, f"decode step, one sequence of about {len(prompt) + tokens} positions")
    for rid in live:
        runner.end(rid)
    return text


def verify(model_dir: str, reference: str, dtype: str = "float32", ctx: Optional[int] = None) -> List[str]:
    """Compares the engine with a reference file of the reference's format (scripts/gen_reference.py:46-79): per case
    the L2 norm of the last prompt token's hidden state after each layer (index 0 = the embedding), then teacher-forced
    steps with the top logits.  Gate (crates/cli/src/verify.rs:15-19): logits within 5e-4 + 1e-4 |ref|, norms within
    1e-4 relative, the greedy token equal.  Returns the list of mismatches (empty = verified)."""
    import torch

    from .engine import Engine, StepEntry

    with open(reference) as fh:
        ref = json.load(fh)
    engine = Engine(model_dir, dtype=dtype, ctx=ctx, max_batch=1, cuda_graphs=False)
    runner = engine.runner
    problems: List[str] = []
    for c, case in enumerate(ref["cases"]):
        ids = list(case["prompt_ids"])
        norms = {}

        def observe(i, hidden, norms=norms):
            norms[i] = float(torch.linalg.vector_norm(hidden[-1]))

        rid = f"verify{c}"
        runner.begin(rid)
        logits = runner.step([StepEntry(rid, ids, [len(ids) - 1])], observe=observe)[0]
        for i, want in enumerate(case.get("layer_norms", [])):
            if abs(norms[i] - want) > 1e-4 * abs(want):
                problems.append(f"case {c}: hidden-state norm at index {i} is {norms[i]:.6f}, reference {want:.6f}")
        for s, step in enumerate(case["steps"]):
            row = logits.float().cpu()
            for token, want in step["top"]:
                got = float(row[token])
                if abs(got - want) > 5e-4 + 1e-4 * abs(want):
                    problems.append(f"case {c} step {s}: logit of token {token} is {got:.6f}, reference {want:.6f}")
            best = int(torch.argmax(row))
            if best != step["token"]:
                problems.append(f"case {c} step {s}: greedy token is {best}, reference {step['token']}")
            logits = runner.step([StepEntry(rid, [step["token"]], [0])])[0]       # teacher forcing
        runner.end(rid)
    return problems


def cmd_verify(args) -> int:
    problems = verify(args.model_dir, args.reference, args.dtype, args.ctx)
    for line in problems[:20]:
        print(line, file=sys.stderr)
    if problems:
        print(f"verify failed: {len(problems)} mismatch(es)", file=sys.stderr)
        return 1
    print("verified: logits, hidden-state norms and greedy tokens match the reference")
    return 0


def cmd_random(args) -> int:
    import torch

    from .config.base import read_json
    from .models import architecture_for
    from .weights import write_random_model

    raw = read_json(args.config)
    config = architecture_for(raw).config_class.from_dict(raw)
    dtype = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    write_random_model(args.out, config, args.seed, dtype)
    print(f"wrote {args.out}/config.json and model.safetensors ({args.dtype}, seed {args.seed})")
    return 0


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    common = argparse.ArgumentParser(add_help=False)
    common.add_argument("--ctx", type=int, default=None, help="context window: prompt plus reply [default: 2048 or the model's maximum]")
    common.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    if argv and argv[0] in ("bench", "verify", "random"):
        ap = argparse.ArgumentParser(prog=f"marin-run {argv[0]}", parents=[common])
        if argv[0] == "bench":
            ap.add_argument("model_dir")
            ap.add_argument("--prompt-tokens", type=int, default=128)
            ap.add_argument("--tokens", type=int, default=64)
            ap.add_argument("--runs", type=int, default=3)
            ap.add_argument("--warmup", type=int, default=1)
            ap.add_argument("--json", default=None)
            ap.add_argument("--profile", action="store_true", help="also print where a step's time goes, stage by stage")
            _add_sampling(ap, temp=0.0, top_p=1.0)
            return cmd_bench(ap.parse_args(argv[1:]))
        if argv[0] == "verify":
            ap.add_argument("model_dir")
            ap.add_argument("--reference", required=True)
            ap.set_defaults(dtype="float32")
            return cmd_verify(ap.parse_args(argv[1:]))
        ap.add_argument("--config", required=True)
        ap.add_argument("--seed", type=int, default=0)
        ap.add_argument("--out", required=True)
        return cmd_random(ap.parse_args(argv[1:]))
    ap = argparse.ArgumentParser(prog="marin-run", parents=[common], description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("model_dir")
    ap.add_argument("-p", "--prompt", default=None, help="complete this text once and exit")
    ap.add_argument("--prompt-ids", default=None, help="token ids of the prompt, separated by commas or spaces")
    ap.add_argument("--max-tokens", type=int, default=DEFAULT_MAX_TOKENS)
    ap.add_argument("--metrics", action="store_true", help="print where the time went after the reply")
    _add_sampling(ap, temp=0.7, top_p=0.9)
    return cmd_run(ap.parse_args(argv))


if __name__ == "__main__":
    sys.exit(main())
