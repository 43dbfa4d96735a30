#!/usr/bin/env python
"""Throughput of the tcgen05 bf16 GEMM against the vendor library on the same shapes.

Each shape is timed with CUDA events over back-to-back launches after warm-up; the
operands (tens to hundreds of MB) are rotated so that consecutive launches do not
reuse L2-resident data.  Reports TFLOP/s and the fraction of the measured cuBLAS
bf16 peak (``MEASURED_PEAKS.json``).

    python benchmarks/microbench_gemm.py [--only M,N,K] [--iters 20] [--warmup 5] [--no-library]
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

SHAPES = [  # (M, N, K, a_t, b_t)
    (2048, 6144, 2560, False, False), (2048, 19456, 2560, False, False), (2048, 2560, 9728, False, False),
    (4096, 6144, 4096, False, False), (4096, 28672, 4096, False, False), (8192, 8192, 8192, False, False),
    (4096, 4096, 4096, False, True), (4096, 4096, 4096, True, True), (2048, 151936, 2560, False, False),
]
# every product of one Llama-3-8B step at 4096 tokens per GPU: forward (NT), input gradient (NN),
# weight gradient (TN)
LLAMA = [
    (4096, 6144, 4096, False, False), (4096, 4096, 4096, False, False), (4096, 28672, 4096, False, False),
    (4096, 4096, 14336, False, False), (4096, 128256, 4096, False, False),
    (4096, 14336, 4096, False, True), (4096, 4096, 28672, False, True), (4096, 4096, 6144, False, True),
    (4096, 4096, 128256, False, True),
    (4096, 14336, 4096, True, True), (28672, 4096, 4096, True, True), (6144, 4096, 4096, True, True),
    (4096, 4096, 4096, True, True), (128256, 4096, 4096, True, True),
]


def peak_tflops() -> float:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["bf16_tflops"])
    return 1590.0


def time_fn(fn, n_rot, iters=20, warmup=5):
    for i in range(warmup):
        fn(i % n_rot)
    torch.cuda.synchronize()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(i % n_rot)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    from gefen_x_b200.ops import tcgemm

    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="", help="M,N,K: time only this shape (NT)")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--no-library", action="store_true", help="skip the vendor-library timing")
    ap.add_argument("--set", default="models", choices=("models", "llama"), help="shape list")
    ap.add_argument("--kernel", default="pair", choices=("pair", "single"),
                    help="pair: CTA-pair kernel where eligible (default); single: single-CTA kernel only")
    ap.add_argument("--bn", type=int, default=0, help="force the pair kernel's tile width (128 / 256)")
    ap.add_argument("--sustained", type=float, default=0.0,
                    help="seconds: time each implementation back to back for this long under the power cap "
                         "(with the clocks sampled) instead of a short burst")
    args = ap.parse_args()
    tcgemm.set_pair_kernel(args.kernel == "pair", args.bn)
    shapes = LLAMA if args.set == "llama" else SHAPES
    if args.only:
        m, n, k = (int(v) for v in args.only.split(","))
        shapes = [(m, n, k, False, False)]
    dev = torch.device("cuda", 0)
    peak = peak_tflops()
    for m, n, k, a_t, b_t in shapes:
        n_rot = 3 if (m * k + n * k) * 2 < (1 << 30) else 2
        a = [torch.randn((k, m) if a_t else (m, k), device=dev).bfloat16() for _ in range(n_rot)]
        b = [torch.randn((k, n) if b_t else (n, k), device=dev).bfloat16() for _ in range(n_rot)]
        out = torch.empty(m, n, device=dev, dtype=torch.bfloat16)

        def ours(i):
            tcgemm.gemm(a[i], b[i], a_t=a_t, b_t=b_t, out=out)

        def lib(i):
            x = a[i].t() if a_t else a[i]
            y = b[i] if b_t else b[i].t()
            torch.matmul(x, y, out=out)

        if args.sustained > 0:
            from gefen_x_b200.utils.clocks import ClockSampler

            for name, fn in (("library", lib), ("ours", ours), ("library", lib), ("ours", ours)):
                burst = time_fn(fn, n_rot, 5, 3)
                iters = max(10, int(args.sustained * 1e3 / burst))
                cs = ClockSampler(0, 100)
                cs.start()
                t = time_fn(fn, n_rot, iters, 0)
                clk = cs.stop()
                print(json.dumps({"M": m, "N": n, "K": k, "a_t": a_t, "b_t": b_t, "impl": name, "sustained_s": args.sustained,
                                  "ms": t, "tflops": 2.0 * m * n * k / t / 1e9, "burst_ms": burst, "clocks": clk}),
                      flush=True)
            continue
        t_ours = time_fn(ours, n_rot, args.iters, args.warmup)
        t_lib = float("nan") if args.no_library else time_fn(lib, n_rot, args.iters, args.warmup)
        flops = 2.0 * m * n * k
        print(json.dumps({"M": m, "N": n, "K": k, "a_t": a_t, "b_t": b_t, "kernel": args.kernel, "bn": args.bn,
                          "ours_ms": t_ours, "ours_tflops": flops / t_ours / 1e9,
                          "ours_fraction_of_measured_peak": flops / t_ours / 1e9 / peak,
                          "library_ms": t_lib, "library_tflops": flops / t_lib / 1e9}), flush=True)
        del a, b, out
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
