"""Where the roles of the persistent matrix product spend their time: ``python -m marin_b200.kernels.probe``.

Builds the tensor-core library with ``-DTC_PROBE`` (a copy beside the normal one: the define is part of the library's
name), runs one many-token product tile by tile and prints, per k-block of 64, the clock ticks the TMA producer waited
for a free stage and spent issuing, and the ticks the MMA thread waited for a full stage and for a free accumulator.
The MMAs of a k-block of a 128 x bn tile take 2 * bn ticks on the tensor core; what the MMA thread's loop takes beyond
that is what the feeding costs.  A measuring tool: nothing in the engine uses this build.
"""
from __future__ import annotations

import argparse
import ctypes
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--rows", type=int, default=18944, help="weight rows N (default: 148 tiles of 128)")
    ap.add_argument("--width", type=int, default=2560, help="K")
    ap.add_argument("--tile", type=int, default=256, help="tokens per tile (a multiple of 16 from 128 to 256)")
    ap.add_argument("--ctas", type=int, default=0, help="CTAs at work (default: one per SM)")
    args = ap.parse_args(argv)
    defines = [d for d in os.environ.get("MARIN_B200_DEFINES", "").split(",") if d and d != "TC_PROBE"]
    os.environ["MARIN_B200_DEFINES"] = ",".join(defines + ["TC_PROBE"])

    import torch

    from . import ops

    dev = torch.device("cuda:0")
    lib = ops._lib("mb_gemm_tc")
    T, N, K, bn = args.tokens, args.rows, args.width, args.tile
    ctas = args.ctas or ops.SM_COUNT
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn(T, K, device=dev, generator=g).to(torch.bfloat16)
    w = torch.randn(N, K, device=dev, generator=g).to(torch.bfloat16)
    out = torch.empty(T, N, device=dev, dtype=torch.bfloat16)
    scratch = ops._scratch_for(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def run():
        rc = lib.mb_gemm_tc_persistent(ops._ptr(x), ops._ptr(w), ops._ptr(out), 0, T, N, K, bn, ctas, ops._ptr(scratch.error), ops._stream())
        if rc:
            raise SystemExit(f"the launch was refused ({rc})")

    for _ in range(3):
        run()
    best = None
    for _ in range(8):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        run()
        b.record()
        torch.cuda.synchronize()
        best = a.elapsed_time(b) if best is None else min(best, a.elapsed_time(b))
    ops.check_device_errors()
    ticks = (ctypes.c_longlong * (148 * 8))()
    if lib.mb_gemm_tc_probe_read(ticks):
        raise SystemExit("the probe's counters could not be read")
    tiles = -(-N // 128) * -(-T // bn)
    grid = min(tiles, ctas)
    flops = 2.0 * T * N * K
    print(f"{T} tokens x {N} rows x {K}, tiles of 128 x {bn}, {grid} CTAs: {best * 1e3:.1f} us, {flops / best / 1e9:.0f} TFLOP/s "
          f"({flops / best / 1e9 / grid:.2f} per SM at work); the MMAs of a k-block take {2 * bn} ticks")
    print("CTA   k-blocks   producer: waits  issues   MMA thread: waits for a stage  for an accumulator  whole loop   (ticks per k-block)")
    for cta in sorted({0, grid // 2, grid - 1}):
        kblocks = len(range(cta, tiles, grid)) * -(-K // 64)
        v = [ticks[cta * 8 + i] / max(kblocks, 1) for i in range(5)]
        print(f"{cta:3d}   {kblocks:8d}   {v[0]:15.0f}  {v[1]:6.0f}   {v[2]:29.0f}  {v[3]:18.0f}  {v[4]:10.0f}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
