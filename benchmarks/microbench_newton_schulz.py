#!/usr/bin/env python
"""Newton–Schulz orthogonalisation (the Muon inner loop) on one GPU.

Times five quintic iterations on Llama-3-8B matrix shapes with CUDA events after warm-up, over
rotating inputs: the bf16 iterations on the own tcgen05 GEMM, the same iterations through the
library (``torch.matmul``), and the e4m3 iterations (``fp8_ns``) on the own kind::f8f6f4 GEMM and on
the library's row-scaled fp8 GEMM.  FLOPs per iteration for an
oriented ``[m, n]`` (m <= n): ``2 m^2 n`` (Gram) + ``2 m^3`` (Gram squared) + ``2 m^2 n`` (update).

    python benchmarks/microbench_newton_schulz.py [--iters 5] [--shapes 4096x4096,4096x14336]
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    from gefen_x_b200.optim import newton_schulz as NS

    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--shapes", default="4096x4096,4096x14336,1024x4096")
    ap.add_argument("--breakdown", action="store_true", help="also time the pieces of one e4m3 iteration")
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    sched = NS.normalize_schedule(None, 5)

    def library(x):
        for a, b, c in sched:
            g = x @ x.t()
            u = torch.addmm(g, g, g, beta=b, alpha=c)
            x = torch.addmm(x, u, x, beta=a)
        return x

    for spec in args.shapes.split(","):
        m, n = sorted(int(v) for v in spec.split("x"))
        xs = [torch.randn(m, n, device=dev).bfloat16() for _ in range(3)]
        xs = [x / x.norm() for x in xs]
        flops = len(sched) * (4.0 * m * m * n + 2.0 * m ** 3)

        def timed(name, fn):
            for i in range(args.warmup):
                fn(xs[i % 3])
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(args.iters):
                fn(xs[i % 3])
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / args.iters
            print(json.dumps({"shape": [m, n], "path": name, "ms": ms, "tflops": flops / ms / 1e9}), flush=True)

        timed("bf16, own tcgen05 GEMM", lambda x: NS._iterate(x, sched))
        timed("bf16, library matmul", library)
        if NS.fp8_applies((m, n), True) and NS.fp8_supported(dev):
            NS.set_fp8_gemm("tcgen05")
            timed("e4m3, own tcgen05 kind::f8f6f4 GEMM", lambda x: NS._iterate_fp8(x, sched))
            NS.set_fp8_gemm("library")
            timed("e4m3, library row-scaled GEMM", lambda x: NS._iterate_fp8(x, sched))
            NS.set_fp8_gemm("tcgen05")
            if args.breakdown:
                from gefen_x_b200.ops.quant import quantize_cols_e4m3_t as quant_t, quantize_rows_e4m3 as quant

                flops = 1.0
                x2 = torch.randn(m, n, device=dev).bfloat16()
                g = torch.randn(m, m, device=dev).bfloat16()
                xq, sx, _ = quant(xs[0])
                gq, sg, _ = quant(g)
                xtq, sxt = quant_t(xs[0])
                timed("piece: quantise X", lambda x: quant(x))
                timed("piece: quantise a X + U X, write X", lambda x: quant(x, x2, 3.4, 1.0, want_y=True))
                timed("piece: quantise X by columns, transposed", lambda x: quant_t(x))
                timed("piece: quantise b G + c G G", lambda x: quant(g, g, -4.7, 2.0))
                for backend in ("tcgen05", "library"):
                    NS.set_fp8_gemm(backend)
                    timed("piece: fp8 GEMM X X^T ({})".format(backend), lambda x: NS._mm_fp8(xq, sx, xq, sx))
                    timed("piece: fp8 GEMM G G ({})".format(backend), lambda x: NS._mm_fp8(gq, sg, gq, sg))
                    timed("piece: fp8 GEMM U X ({})".format(backend), lambda x: NS._mm_fp8(gq, sg, xtq, sxt))
                NS.set_fp8_gemm("tcgen05")


if __name__ == "__main__":
    main()
