"""Where a step's time goes, stage by stage: every kernel of a step with its time inside the step, the bytes it has
to move and the flops it has to do, and what fraction of the device's peaks that is.

The reference times its stages with events around each (crates/model/src/qwen3/gpu_probe.rs:8-55,
crates/metrics/src/stage.rs:5-19; ``marin-run bench --profile``).  Here kernels overlap by design (each is launched
as a programmatic dependent of the one before and starts its own prologue and weight fetches while that one ends), so
events between them would measure another program.  Instead the steps run exactly as they do in serving (replayed
graphs for single-token steps) under the CUDA profiling interface (``torch.profiler``, kernel activity records
only), and a kernel's *share* of the step is the time from the end of the kernel before it to its own end: shares
add up to the step's time.  Each launch brings its own label and cost (``ops.launch_log``); attention's part that
grows with the cache is scaled with the lengths of the profiled step.

Numbers taken under the profiler are for the breakdown only: throughput is measured without it (``bench.py``).
"""
from __future__ import annotations

import statistics
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence

import torch

from ..kernels import ops
from .step import Runner, StepEntry


@dataclass
class StageRow:
    stage: str
    kernel: str
    calls: int              # launches per step
    share_us: float         # per step: sum over the calls of (end - end of the kernel before)
    busy_us: float          # per step: sum of the kernels' own durations (they overlap their neighbours)
    bytes: float            # per step, as the algorithm needs them
    flops: float

    def gbs(self) -> float:
        return self.bytes / (self.share_us * 1e-6) / 1e9 if self.share_us > 0 else 0.0

    def tflops(self) -> float:
        return self.flops / (self.share_us * 1e-6) / 1e12 if self.share_us > 0 else 0.0


def lengths_of(runner: Runner, entries: Sequence[StepEntry]):
    """Keys read and (query, key) pairs of the single-token rows and of the portions of a step that is about to run."""
    counts = {"decode": [0, 0], "prefill": [0, 0]}
    for e in entries:
        before, n = runner.length(e.req_id), len(e.tokens)
        which = counts["decode" if n == 1 else "prefill"]
        which[0] += before + n
        which[1] += n * before + n * (n + 1) // 2
    total = [counts["decode"][0] + counts["prefill"][0], counts["decode"][1] + counts["prefill"][1]]
    return {"decode": counts["decode"], "prefill": counts["prefill"], "all": total}


def _kernel_events(prof) -> List:
    events = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA
              and not e.name.lower().startswith(("memcpy", "memset"))]
    events.sort(key=lambda e: e.time_range.end)
    return events


def profile_steps(runner: Runner, make_entries: Callable[[int], Sequence[StepEntry]], steps: int = 4, warmup: int = 3,
                  after_step: Optional[Callable[[torch.Tensor], None]] = None) -> List[StageRow]:
    """Runs ``warmup + steps`` steps (``make_entries(i)`` gives step i's entries; every step must launch the same
    kernels) and returns the stages of one step in launch order, times as medians over the profiled steps.
    ``after_step(logits)`` runs after each step inside the profiled region (sampling, for steps that do not carry it)."""
    from torch.profiler import ProfilerActivity, profile

    def one(i, log=None):
        entries = make_entries(i)
        sizes = lengths_of(runner, entries)
        ops.launch_log = log
        try:
            logits = runner.step(entries)
            if after_step is not None:
                with ops.using(runner.scratch):
                    after_step(logits)
        finally:
            ops.launch_log = None
        return sizes

    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    labels: List[dict] = []
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for i in range(steps):
            log: List[dict] = []
            sizes = one(warmup + i, log)
            replayed = runner._replayed
            if replayed is not None:                        # a graph brings the labels recorded at its capture
                log = [dict(entry) for entry in replayed["labels"]] + log
            labels = log
        torch.cuda.synchronize()
    events = _kernel_events(prof)
    per_step = len(labels)
    if per_step == 0 or len(events) != per_step * steps:
        raise RuntimeError(f"{len(events)} kernels were recorded over {steps} steps but a step launches {per_step}: "
                           "the steps did not launch the same kernels, or kernels of another library ran among them")
    shares = [[] for _ in range(per_step)]
    busy = [[] for _ in range(per_step)]
    gaps = []
    for s in range(1 if steps > 1 else 0, steps):            # the first profiled step has no kernel before it
        for k in range(per_step):
            e = events[s * per_step + k]
            busy[k].append(e.time_range.end - e.time_range.start)
            if k == 0:
                # the step's first kernel has nothing of this step ahead of it: its share is its own duration, and
                # the idle time since the last step's end (the host's work between two steps) is a row of its own
                shares[k].append(e.time_range.end - e.time_range.start)
                if s > 0:
                    gaps.append(max(0.0, e.time_range.start - events[s * per_step - 1].time_range.end))
            else:
                shares[k].append(max(0.0, e.time_range.end - events[s * per_step + k - 1].time_range.end))
    rows: List[StageRow] = []
    merged: Dict[tuple, StageRow] = {}
    if gaps:
        rows.append(StageRow("(between steps)", "the device idle: host work, launch", 0, statistics.median(gaps), 0.0, 0.0, 0.0))
    for k, entry in enumerate(labels):
        keys, pairs = sizes.get(entry.get("rows", "all"), sizes["all"])
        nbytes = entry["bytes"] + entry["bytes_per_key"] * keys
        flops = entry["flops"] + entry["flops_per_pair"] * pairs
        key = (entry["stage"], entry["kernel"])
        row = merged.get(key)
        if row is None:
            row = merged[key] = StageRow(entry["stage"], entry["kernel"], 0, 0.0, 0.0, 0.0, 0.0)
            rows.append(row)
        row.calls += 1
        row.share_us += statistics.median(shares[k])
        row.busy_us += statistics.median(busy[k])
        row.bytes += nbytes
        row.flops += flops
    return rows


def format_table(rows: Sequence[StageRow], hbm_gbs: float, peak_tflops: float, title: str = "") -> str:
    """The stages as a text table; fractions are of the given peaks (a copy's bandwidth, a library product's rate)."""
    total = sum(r.share_us for r in rows)
    lines = []
    if title:
        lines.append(title)
    lines.append(f"{'stage':18s} {'kernel':44s} {'calls':>5s} {'in step us':>10s} {'%':>5s} {'busy us':>8s} {'MB':>9s} {'GB/s':>7s} "
                 f"{'of HBM':>6s} {'GFLOP':>9s} {'TFLOP/s':>8s} {'of peak':>7s}")
    for r in rows:
        lines.append(f"{r.stage[:18]:18s} {r.kernel[:44]:44s} {r.calls:5d} {r.share_us:10.1f} {100 * r.share_us / total if total else 0:5.1f} "
                     f"{r.busy_us:8.1f} {r.bytes / 1e6:9.2f} {r.gbs():7.0f} {100 * r.gbs() / hbm_gbs:5.1f}% {r.flops / 1e9:9.2f} "
                     f"{r.tflops():8.1f} {100 * r.tflops() / peak_tflops:6.1f}%")
    nbytes, flops = sum(r.bytes for r in rows), sum(r.flops for r in rows)
    lines.append(f"{'step':18s} {'':44s} {sum(r.calls for r in rows):5d} {total:10.1f} {100.0:5.1f} {sum(r.busy_us for r in rows):8.1f} "
                 f"{nbytes / 1e6:9.2f} {nbytes / (total * 1e-6) / 1e9 if total else 0:7.0f} "
                 f"{100 * nbytes / (total * 1e-6) / 1e9 / hbm_gbs if total else 0:5.1f}% {flops / 1e9:9.2f} "
                 f"{flops / (total * 1e-6) / 1e12 if total else 0:8.1f} {100 * flops / (total * 1e-6) / 1e12 / peak_tflops if total else 0:6.1f}%")
    return "\n".join(lines)
