#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, with their fractions of roofline.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers N] [--impl ours|reference]

The default run has the layer sizes of the Qwen3-4B layout with random bfloat16 weights, a batch of 8
sequences and a context of 4096 positions (the last timed step reaches it).  A "step" is one decode
step.  One JSON line is printed:

  value      decoded tokens a second, K steps timed on the device with CUDA events
  e2e        the same through the Python entry point (Engine.step): every step the host packs and sends the next
             step's inputs from pinned memory and reads the sampled ids back (the step after the running one is
             launched before those ids have arrived: its token ids are fed on the device)
  prefill    one 2,048-token prompt in one step: tokens a second and the fraction of the bf16 peak
  roofline   bytes a decode step has to read (every weight once, the cache of the live requests) / its time
  points     decode at batch 1 and 64

Peaks come from MEASURED_PEAKS.json beside this file if present, else 6.65 TB/s and 1.59 PFLOP/s.
Between timed iterations nothing is flushed: a decode step reads gigabytes of weights, far more than the
126 MB L2 holds (config.l2 says so).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_4B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 36, "hidden_size": 2560,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 9728,
    "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 40960,
}
QWEN3_8B = dict(QWEN3_4B, hidden_size=4096, intermediate_size=12288, tie_word_embeddings=False)
QWEN3_14B = dict(QWEN3_4B, num_hidden_layers=40, hidden_size=5120, num_attention_heads=40, intermediate_size=17408,
                 tie_word_embeddings=False)
LAYOUTS = {"4b": QWEN3_4B, "8b": QWEN3_8B, "14b": QWEN3_14B}
CONTEXT = 4096
PREFILL_TOKENS = 2048
PAGE = 16
PUBLISHED = None     # the reference published no number for this metric on this configuration


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs (reads only)."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu="0"):
        self.rows, self.proc, self.gpu = [], None, str(gpu)

    @staticmethod
    def gpu_in_use():
        """What nvidia-smi should be asked about: the device this process computes on (its UUID), not index 0 of the
        box, which may be another job's GPU."""
        import torch

        try:
            uuid = str(torch.cuda.get_device_properties(torch.cuda.current_device()).uuid)
            return uuid if uuid.startswith("GPU-") else "GPU-" + uuid
        except Exception:  # noqa: BLE001 - an older torch without the field: the first visible device
            visible = os.environ.get("CUDA_VISIBLE_DEVICES", "").split(",")[0].strip()
            return visible or "0"

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", self.gpu, f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, reasons, smax = [], set(), None
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                smax = float(r[1])
            except (ValueError, IndexError):
                continue
            for name, v in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], r[3:7]):
                if v == "Active":
                    reasons.add(name)
        busy = [c for c in sm if smax and c > 0.5 * smax] or sm
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(sm), "samples_under_load": len(busy), "gpu": self.gpu}


def model_bytes_and_flops(engine, batch, tokens):
    """Bytes of weights a decode step of `batch` tokens reads (what the model's parts say they read), and the flops
    of a `tokens`-long prompt with one row of logits (causal: every token looks at itself and what came before)."""
    dtype = engine.rt.dtype
    pairs = tokens * (tokens + 1) // 2
    return engine.model.bytes_read(batch, dtype), engine.model.flops(tokens, pairs, 1)


def kv_bytes_per_token(engine):
    """Bytes one cached position holds over all layers (what a decoded token reads per position of its sequence)."""
    return engine.model.cache_bytes_read(1, engine.rt.dtype)


def fill_cache(engine, seed=1):
    import torch

    g = torch.Generator(device=engine.rt.device).manual_seed(seed)
    for group in engine.cache.groups:
        for t in (group.k, group.v):
            flat = t.view(-1)
            step = 1 << 28
            for at in range(0, flat.numel(), step):
                n = min(step, flat.numel() - at)
                flat[at:at + n] = (torch.randn(n, device=t.device, generator=g, dtype=torch.float32) * 0.5).to(t.dtype)


def decode_device(engine, batch, steps, warmup, context):
    """K decode steps of `batch` sequences timed on the device; the last step reaches `context`."""
    import torch

    from marin_b200.engine import StepEntry
    from marin_b200.kernels import ops

    runner = engine.runner
    start_len = context - (steps + warmup)
    ids = [f"bench{i}" for i in range(batch)]
    for rid in ids:
        runner.begin(rid)
        engine.cache.reserve(rid, start_len)
        engine.cache.commit(rid, start_len)
    vocab = engine.config.vocab_size
    tokens = torch.randint(0, vocab, (batch,), dtype=torch.int32).tolist()
    out = runner.scratch.ids(batch)

    def one_step(tokens):
        logits = runner.step([StepEntry(rid, [tok], [0]) for rid, tok in zip(ids, tokens)])
        if runner.greedy_ids is None:                       # a replayed graph has found the largest logits already
            with ops.using(runner.scratch):
                ops.argmax(logits, vocab, out)

    for _ in range(warmup):
        one_step(tokens)
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches = ops.launches
    begin.record()
    for _ in range(steps):
        one_step(tokens)
    end.record()
    torch.cuda.synchronize()
    ms = begin.elapsed_time(end)
    launched = ops.launches - launches
    for rid in ids:
        runner.end(rid)
    mean_context = context - (steps - 1) / 2.0
    return {"tok_s": batch * steps / (ms / 1e3), "ms_per_step": ms / steps, "launches": launched,
            "mean_context": mean_context}


def decode_e2e(engine, batch, steps, warmup, context):
    """The same through Engine.add_request / Engine.step: host token ids in, sampled ids out, every step."""
    import torch

    from marin_b200 import SamplingParams

    vocab = engine.config.vocab_size
    # the prompts are read in portions under the token budget, one request after another, while the requests
    # that are through already decode: leave room for those tokens so that the timed steps end near `context`
    prefill_steps = -(-batch * context // engine.token_budget) + batch
    prompt_len = context - (steps + warmup) - prefill_steps - 2
    g = torch.Generator().manual_seed(3)
    params = SamplingParams(temperature=0.0, max_tokens=context)
    ids = [engine.add_request(torch.randint(0, vocab, (prompt_len,), generator=g).tolist(), params) for _ in range(batch)]
    produced = {i: 0 for i in ids}
    while min(produced.values()) < 1:                       # prompts (untimed)
        for rid, _ in engine.step():
            produced[rid] += 1
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    got = 0
    for _ in range(steps):
        got += len(engine.step())                           # sampled ids are host ints here
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    for i in ids:
        engine.scheduler.cancel(i)
        engine.forget(i)
    # per step the host sends the packed inputs of the next step without its token ids (those are fed on the device:
    # the step is launched before the host has read the ids of the one before) and reads, from pinned memory that the
    # arg-max kernel writes itself, four ints of status and the sampled ids
    bucket = next(b for b in engine.runner.graph_sizes if b >= batch)
    h2d = 4 * (engine.runner.packed_size(bucket) + 1 - bucket)
    return {"value": got / seconds, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * (4 + batch),
            "tokens": got}


def prefill_device(engine, tokens, runs, warmup):
    import torch

    from marin_b200.engine import StepEntry

    runner = engine.runner
    vocab = engine.config.vocab_size
    prompt = torch.randint(0, vocab, (tokens,), generator=torch.Generator().manual_seed(5)).tolist()
    times = []
    for i in range(warmup + runs):
        runner.begin("prefill")
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        runner.step([StepEntry("prefill", prompt, [tokens - 1])])
        end.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(begin.elapsed_time(end))
        runner.end("prefill")
    return statistics.median(times)


def profile_mode(engine, args, pk):
    """Where the time of a decode step (batch 1, 8 and 64) and of a 2,048-token prompt goes, stage by stage
    (marin_b200/engine/profile.py).  Text to stdout; no JSON line: nothing measured here is a throughput figure."""
    import torch

    from marin_b200.engine import StepEntry
    from marin_b200.engine.profile import format_table, profile_steps
    from marin_b200.kernels import ops

    runner, vocab = engine.runner, engine.config.vocab_size
    layers = len(engine.model.blocks)
    where = f"Qwen3-{args.model.upper()} layout, {layers} of {LAYOUTS[args.model]['num_hidden_layers']} layers, bfloat16, page {PAGE}"
    peaks_line = f"peaks ({pk['source']}): {pk['hbm_gbs']:.0f} GB/s copy, {pk['bf16_tflops']:.0f} TFLOP/s bf16"
    print(f"{where}; {peaks_line}; in-step times under the CUDA profiling interface (medians of 6 steps)\n")
    steps, warmup = 6, 4
    for batch in sorted({1, 8, 64, args.batch}):
        ids = [f"prof{batch}_{i}" for i in range(batch)]
        for rid in ids:
            runner.begin(rid)
            engine.cache.reserve(rid, CONTEXT - steps - warmup)
            engine.cache.commit(rid, CONTEXT - steps - warmup)
        rows = profile_steps(runner, lambda i: [StepEntry(rid, [5 + i], [0]) for rid in ids], steps, warmup)
        print(format_table(rows, pk["hbm_gbs"], pk["bf16_tflops"], f"decode step, batch {batch}, sequences of about {CONTEXT} positions"))
        print()
        for rid in ids:
            runner.end(rid)
    prompt = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=torch.Generator().manual_seed(5)).tolist()
    out = runner.scratch.ids(1)

    def entries(i):
        runner.begin(f"prefill{i}")
        return [StepEntry(f"prefill{i}", prompt, [PREFILL_TOKENS - 1])]

    def after(logits):
        ops.stage_name = "sampling"
        ops.argmax(logits, vocab, out)
        runner.end(next(iter(runner.cache.requests)))

    rows = profile_steps(runner, entries, steps, warmup, after_step=after)
    print(format_table(rows, pk["hbm_gbs"], pk["bf16_tflops"], f"prompt of {PREFILL_TOKENS} tokens in one step"))
    engine.check_device()
    return 0


def reference_arm():
    """The reference is a Rust workspace (cargo, rustc); neither exists in this image, so it cannot be
    built or installed offline, and a pip install of its source tree has nothing to install (no Python package)."""
    print(json.dumps({"impl": "reference", "unavailable": "Kayleexx/marin is a Rust workspace; no cargo/rustc in this image and no Python package to pip-install"}))
    return 0


def main() -> int:
    global CONTEXT
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration has (recorded in config)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--model", default="4b", choices=sorted(LAYOUTS), help="layer sizes: Qwen3-4B (the default), 8B or 14B layout")
    ap.add_argument("--context", type=int, default=CONTEXT, help="context length the last timed decode step reaches (default 4096)")
    ap.add_argument("--profile", action="store_true", help="print where a step's time goes, stage by stage, instead of the JSON line")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    CONTEXT = args.context
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    warmup = max(3, args.warmup)

    import torch

    from marin_b200 import Engine
    from marin_b200.config import Qwen3Config
    from marin_b200.kernels import build

    build.build_all(verbose=False)
    raw = dict(LAYOUTS[args.model])
    full_layers = raw["num_hidden_layers"]
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    cfg = Qwen3Config.from_dict(raw)
    pk = peaks()
    max_batch = args.batch if args.no_points else max(args.batch, 64)
    engine = Engine(config=cfg, seed=0, dtype="bfloat16", ctx=CONTEXT, page_size=PAGE, max_batch=max_batch,
                    token_budget=PREFILL_TOKENS)
    fill_cache(engine)
    if args.profile:
        return profile_mode(engine, args, pk)
    weight_bytes, prefill_flops = model_bytes_and_flops(engine, args.batch, PREFILL_TOKENS)
    kv_tok = kv_bytes_per_token(engine)

    clocks = ClockSampler(ClockSampler.gpu_in_use())
    clocks.start()
    main_run = decode_device(engine, args.batch, args.steps, warmup, CONTEXT)
    # the timed steps last a fraction of a second; the same steps run on (untimed) until the sampler has seen about two
    # seconds of this load, so that the median clock rests on tens of readings
    load_until = time.perf_counter() + 2.0
    while time.perf_counter() < load_until:
        decode_device(engine, args.batch, args.steps, 3, CONTEXT)
    clock_record = clocks.stop()

    step_bytes = weight_bytes + args.batch * main_run["mean_context"] * kv_tok
    achieved = step_bytes / (main_run["ms_per_step"] / 1e3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / pk["hbm_gbs"], 4), "peak_source": pk["source"]}

    prefill_ms = prefill_device(engine, PREFILL_TOKENS, runs=3, warmup=3)
    prefill = {"value": round(PREFILL_TOKENS / (prefill_ms / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(prefill_ms, 3),
               "frac": round(prefill_flops / (prefill_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
               "peak_tflops": pk["bf16_tflops"], "peak_source": pk["source"],
               # the step is 17 ms of back-to-back kernels and is timed several times in a row: beside the burst figure,
               # the same against the library's rate in a seconds-long loop under the power cap
               "frac_of_sustained": round(prefill_flops / (prefill_ms / 1e3) / (pk["bf16_tflops_sustained"] * 1e12), 4),
               "peak_tflops_sustained": pk["bf16_tflops_sustained"]}

    points = {}
    if not args.no_points:
        per_seq = -(-CONTEXT // PAGE)
        for b in (1, 64):
            if engine.num_pages < b * per_seq:               # a long context: the pool that fits the device holds fewer sequences
                points[f"decode_b{b}"] = None
                continue
            r = decode_device(engine, b, min(args.steps, 32), 3, CONTEXT)
            points[f"decode_b{b}"] = round(r["tok_s"], 1)
            bytes_b = model_bytes_and_flops(engine, b, PREFILL_TOKENS)[0] + b * r["mean_context"] * kv_tok
            points[f"decode_b{b}_hbm_frac"] = round(bytes_b / (r["ms_per_step"] / 1e3) / 1e9 / pk["hbm_gbs"], 4)

    e2e = None
    if not args.no_e2e:
        e2e = decode_e2e(engine, args.batch, args.steps, warmup, CONTEXT)
        e2e["value"] = round(e2e["value"], 1)

    line = {
        "metric": f"decode tok/s at batch {args.batch} (Qwen3-{args.model.upper()} layout, context {CONTEXT}); prefill tok/s at 2048 tokens; % of roofline",
        "value": round(main_run["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(main_run["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": PUBLISHED, "dtype": "bf16", "data": "synthetic (uniform random token ids, seeded random weights N(0,0.02))",
        "config": {"model": f"Qwen3-{args.model.upper()} layout", "layers": cfg.num_hidden_layers, "layers_full": full_layers, "hidden": cfg.hidden_size,
                   "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "tied": cfg.tie_word_embeddings,
                   "global_batch": args.batch, "seq_len": CONTEXT, "kv_block": PAGE, "prefill_tokens": PREFILL_TOKENS,
                   "parallelism": "1 GPU", "l2": "inputs larger than L2 (weights read per step exceed 126 MB)",
                   "sampling": "greedy on device"},
        "clocks": clock_record, "gpu_launches": main_run["launches"], "prefill": prefill, "roofline": roofline,
        "points": points, "impl": "ours",
    }
    if e2e is not None:
        line["e2e"] = e2e
    engine.check_device()                # a kernel whose bounded wait gave up would make the numbers above worthless: raise
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
