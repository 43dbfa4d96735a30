#!/usr/bin/env python
"""Causal GQA attention: own kernels against the library SDPA on one GPU.

Shape of one Llama-3-8B layer at 2 x 2048 tokens by default (32 query / 8 KV heads of 128).
Forward: ``flash_fwd_kernel`` (tcgen05, fused) and the GEMM-composed forward; backward: the
GEMM-composed backward with own row kernels.  CUDA-event timings after warm-up over rotating
inputs; FLOPs counted for the causal half (4 * B * nq * S^2 * hd / 2 forward, 2.5x backward).

    python benchmarks/microbench_attention.py [--batch 2] [--seq 2048] [--iters 10] [--only flash]
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    from gefen_x_b200.ops import attention as A

    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--only", default="", help="flash: time only the fused forward (profiling)")
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    B, S, nq, nkv, hd = args.batch, args.seq, args.heads, args.kv_heads, args.head_dim
    n_rot = 3
    qs = [torch.randn(B, S, nq, hd, device=dev).bfloat16() for _ in range(n_rot)]
    ks = [torch.randn(B, S, nkv, hd, device=dev).bfloat16() for _ in range(n_rot)]
    vs = [torch.randn(B, S, nkv, hd, device=dev).bfloat16() for _ in range(n_rot)]
    do = torch.randn(B, S, nq, hd, device=dev).bfloat16()
    fwd_flops = 4.0 * B * nq * S * S * hd / 2
    bwd_flops = 2.5 * fwd_flops

    def timed(name, fn, flops):
        for i in range(args.warmup):
            fn(i % n_rot)
        torch.cuda.synchronize()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.iters):
            fn(i % n_rot)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.iters
        print(json.dumps({"kernel": name, "ms": ms, "tflops_causal": flops / ms / 1e9}), flush=True)

    timed("own forward, fused (flash_fwd_kernel, incl. head-major repacking)",
          lambda i: A.attention_fwd(qs[i], ks[i], vs[i], flash=True), fwd_flops)
    if args.only == "flash":
        return
    timed("own forward, GEMM-composed", lambda i: A.attention_fwd(qs[i], ks[i], vs[i], flash=False), fwd_flops)
    ctxs = [A.attention_fwd(qs[i], ks[i], vs[i])[1] for i in range(n_rot)]
    timed("own backward, GEMM-composed", lambda i: A.attention_bwd(ctxs[i], do), bwd_flops)

    def sdpa_fwd(i):
        return F.scaled_dot_product_attention(qs[i].transpose(1, 2), ks[i].transpose(1, 2), vs[i].transpose(1, 2),
                                              is_causal=True, enable_gqa=nq != nkv)

    timed("library SDPA forward", sdpa_fwd, fwd_flops)
    leaves = [(qs[i].clone().requires_grad_(), ks[i].clone().requires_grad_(), vs[i].clone().requires_grad_())
              for i in range(n_rot)]
    outs = [F.scaled_dot_product_attention(a.transpose(1, 2), b.transpose(1, 2), c.transpose(1, 2), is_causal=True,
                                           enable_gqa=nq != nkv) for a, b, c in leaves]
    dot = do.transpose(1, 2)
    timed("library SDPA backward",
          lambda i: torch.autograd.grad(outs[i], leaves[i], dot, retain_graph=True), bwd_flops)


if __name__ == "__main__":
    main()
