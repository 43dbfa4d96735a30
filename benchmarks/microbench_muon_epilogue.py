#!/usr/bin/env python
"""NorMuon + cautious mask + parameter update on one GPU: the three-launch kernels of
``csrc/muon_ops.cu`` against the chain of torch ops they replace.

CUDA events after warm-up, L2 flushed between iterations, Llama-3-8B matrix shapes.  Algorithmic
traffic of the kernels: pass 1 reads the update and the gradient, pass 3 reads update, gradient and
parameter and writes update and parameter (14 bytes per bf16 element with everything on).

    python benchmarks/microbench_muon_epilogue.py [--iters 10] [--shapes 4096x4096,4096x14336]
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
    from gefen_x_b200.ops._ext import ops
    from gefen_x_b200.optim.muon import cautious_mask_

    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--shapes", default="4096x4096,4096x14336")
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    beta2, eps, lr_ratio, wdf = 0.95, 1e-8, 3e-3, 0.9997
    for spec in args.shapes.split(","):
        rows, cols = (int(v) for v in spec.split("x"))
        u0 = (torch.randn(rows, cols, device=dev) * 0.3).bfloat16()
        gr = torch.randn(rows, cols, device=dev).bfloat16()
        p = (torch.randn(rows, cols, device=dev) * 0.05).bfloat16()
        v = torch.zeros(rows, 1, dtype=torch.float32, device=dev)
        scal = torch.tensor([1 - beta2, lr_ratio, wdf], dtype=torch.float32, device=dev)

        def kernels():
            u = u0.clone()
            ops().muon_epilogue(u, gr, v, p, scal, True, True, beta2, eps)

        def torch_chain():
            u = u0.clone()
            row_norm = torch.linalg.vector_norm(u, dim=1, keepdim=True, dtype=torch.float32)
            row_sq = row_norm.square()
            v.mul_(beta2).add_(row_sq, alpha=(1 - beta2) / cols)
            denom = (v / (1 - beta2)).sqrt_().add_(eps)
            frob = row_sq.sum().sqrt_() / torch.linalg.vector_norm(row_norm / denom).clamp(min=1e-38)
            u.mul_((frob / denom).to(u.dtype))
            u = cautious_mask_(u, gr)
            p.mul_(wdf)
            p.add_(u, alpha=-lr_ratio)

        def clone_only():
            u0.clone()

        out = {}
        for name, fn in (("clone only", clone_only), ("kernels", kernels), ("torch chain", torch_chain)):
            ts = []
            for i in range(args.warmup + args.iters):
                flush.fill_(i & 0xFF)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                if i >= args.warmup:
                    ts.append(e0.elapsed_time(e1))
            ts.sort()
            out[name] = ts[len(ts) // 2]
        base = out["clone only"]
        n = rows * cols
        print(json.dumps({"shape": [rows, cols], "kernels_ms": out["kernels"] - base,
                          "torch_chain_ms": out["torch chain"] - base,
                          "kernels_gbs": 14.0 * n / (out["kernels"] - base) / 1e6,
                          "speedup": (out["torch chain"] - base) / (out["kernels"] - base)}), flush=True)


if __name__ == "__main__":
    main()
