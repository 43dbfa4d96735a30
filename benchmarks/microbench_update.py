#!/usr/bin/env python
"""Optimizer-step microbenchmark on one GPU (bf16 parameters).

Shapes: one flat 1-D tensor and the matrices [4096x4096], [4096x14336],
[14336x4096], [128256x4096]; gradients i.i.d. N(0, 1e-3).  For every shape the
fused update (codebook momentum + factored second moment for matrices, block
second moment for the flat tensor) is timed with CUDA events after warm-up, with
a buffer larger than L2 written between iterations, and reported as step
milliseconds and as the fraction of the HBM roofline (algorithmic bytes / measured
copy bandwidth).  ``--impl reference`` times the reference package installed in
``baseline/_ref`` the same way (its own harness: reference
``benchmarks/microbench/microbench_v1v2.py:36-47``).

    python benchmarks/microbench_update.py [--impl ours|reference] [--iters 20]
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

SHAPES = [("flat", (16 * 1024 * 1024,)), ("4096x4096", (4096, 4096)), ("4096x14336", (4096, 14336)),
          ("14336x4096", (14336, 4096)), ("128256x4096", (128256, 4096))]


def measured_hbm_gbs() -> float:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"])
    return 6650.0


def algorithmic_bytes(shape, factored: bool) -> int:
    """Bytes an ideal implementation moves: grad (2) + idx (1) read for the statistics, then
    grad (2) + idx (1) + param (2) read and idx (1) + param (2) written: 11 B/element;
    the one-pass block path needs 8 B/element (its second pass hits cache)."""
    n = 1
    for s in shape:
        n *= s
    return n * (11 if factored else 8)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--shapes", default="")
    ap.add_argument("--wide", action="store_true",
                    help="ours: streamed kernels with 16 instead of 8 elements per thread")
    ap.add_argument("--no-streaming", action="store_true",
                    help="ours: the register-pipelined fast kernels instead of the streamed ones")
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    if args.impl == "reference":
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
        os.environ.setdefault("GEFEN_KERNEL_BUILD_ROOT", os.path.join(ROOT, "baseline", "_ref_build"))
        os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
        from gefen import Gefen
    else:
        from gefen_x_b200 import Gefen
        from gefen_x_b200.ops import update as _update

        _update.set_streaming(not args.no_streaming)
        _update.set_wide_chunks(args.wide)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)   # 2x the 126 MB L2
    # A few milliseconds of device work queued ahead of every timed step, so that the host
    # has enqueued the whole step before the device reaches the first event (the events
    # then bracket device time only, not launch latency).
    blocker = torch.randn(8192, 8192, device=dev, dtype=torch.bfloat16)
    peak = measured_hbm_gbs()
    results = []
    wanted = set(args.shapes.split(",")) if args.shapes else None
    for name, shape in SHAPES:
        if wanted and name not in wanted:
            continue
        g = torch.Generator(device=dev).manual_seed(0)
        p = (torch.randn(shape, device=dev, generator=g) * 0.02).bfloat16().requires_grad_()
        grads = [(torch.randn(shape, device=dev, generator=g) * 1e-3).bfloat16() for _ in range(2)]
        opt = Gefen([(name, p)], lr=1e-4, weight_decay=0.01)
        times = []
        for i in range(args.warmup + args.iters):
            p.grad = grads[i % 2]
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            torch.mm(blocker, blocker)
            torch.mm(blocker, blocker)
            flush.fill_(i & 0xFF)
            e0.record()
            opt.step()
            e1.record()
            torch.cuda.synchronize()
            if i >= args.warmup:
                times.append(e0.elapsed_time(e1))
        times.sort()
        med = times[len(times) // 2]
        factored = len(shape) == 2
        nbytes = algorithmic_bytes(shape, factored)
        st = opt.state[p]
        state_bytes = sum(v.numel() * v.element_size() for v in st.values() if torch.is_tensor(v))
        rec = {"shape": name, "impl": args.impl, "ms_median": med, "ms_min": times[0],
               "gbs": nbytes / med / 1e6, "hbm_fraction_of_measured": nbytes / med / 1e6 / peak,
               "period": int(st["automatic_period"]),
               "plan_fast": sorted({pl.fast for pl in opt._plan_cache._plans.values()}) if args.impl == "ours" else None, "state_bytes_per_param": state_bytes / p.numel()}
        results.append(rec)
        print(json.dumps(rec), flush=True)
        del opt, p, grads
        torch.cuda.empty_cache()
    return results


if __name__ == "__main__":
    main()
