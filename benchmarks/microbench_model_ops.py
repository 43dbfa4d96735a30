#!/usr/bin/env python
"""Device time and HBM-roofline fraction of the model kernels and of the peer-memory kernels.

Shapes of one Llama-3-8B layer at 4096 tokens (hidden 4096, FFN 14336, 32 query / 8 KV heads of
128, vocabulary 128256 cut to ``--vocab``).  Every kernel is timed with CUDA events after
warm-up with a buffer larger than L2 written between iterations; the fraction is algorithmic
bytes / time / measured copy bandwidth (``MEASURED_PEAKS.json``).  The peer-memory kernels
(``gather_kernel``, ``reduce_segments_kernel``) run here on local buffers standing in for the
peers' arenas (one GPU): what is measured is their HBM-side efficiency, not NVLink.

    python benchmarks/microbench_model_ops.py [--iters 10] [--only rmsnorm,rope,swiglu,xent,comm]
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def measured_hbm_gbs() -> float:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"])
    return 6650.0


class _GatherSeg(ctypes.Structure):
    _fields_ = [("src_off", ctypes.c_longlong), ("dst_off", ctypes.c_longlong),
                ("src_rank", ctypes.c_int), ("pad", ctypes.c_int)]


class _ReduceSeg(ctypes.Structure):
    _fields_ = [("dst", ctypes.c_void_p), ("src", ctypes.c_void_p * 8)]


def main():
    from gefen_x_b200.ops import model as M
    from gefen_x_b200.ops._ext import ops

    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--vocab", type=int, default=32064, help="columns of the logits (a quarter of 128256)")
    ap.add_argument("--only", default="")
    args = ap.parse_args()
    only = set(args.only.split(",")) if args.only else None
    dev = torch.device("cuda", 0)
    peak = measured_hbm_gbs()
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    T, H, F, NH, NKV, HD = args.tokens, 4096, 14336, 32, 8, 128
    bf = torch.bfloat16

    def timed(name, fn, nbytes):
        ts = []
        for i in range(args.warmup + args.iters):
            flush.fill_(i & 0xFF)
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if i >= args.warmup:
                ts.append(e0.elapsed_time(e1))
        ts.sort()
        med = ts[len(ts) // 2]
        print(json.dumps({"kernel": name, "ms_median": med, "algorithmic_mb": nbytes / 1e6,
                          "gbs": nbytes / med / 1e6, "hbm_fraction_of_measured": nbytes / med / 1e6 / peak}),
              flush=True)

    if only is None or "rmsnorm" in only:
        x = torch.randn(T, H, device=dev).to(bf)
        w = torch.randn(H, device=dev).to(bf)
        dy = torch.randn(T, H, device=dev).to(bf)
        y, rstd = M.rmsnorm_fwd(x, w, 1e-5)
        timed("rmsnorm_fwd", lambda: M.rmsnorm_fwd(x, w, 1e-5), 2 * T * H * 2)
        timed("rmsnorm_bwd", lambda: M.rmsnorm_bwd(dy, x, w, rstd), 3 * T * H * 2)
    if only is None or "rope" in only:
        q = torch.randn(2, T // 2, NH, HD, device=dev).to(bf)
        cos, sin = M.rope_tables(T // 2, HD, 5e5, dev)
        timed("rope", lambda: M.rope_(q, cos, sin), 2 * q.numel() * 2)
    if only is None or "swiglu" in only:
        gu = torch.randn(T, 2 * F, device=dev).to(bf)
        do = torch.randn(T, F, device=dev).to(bf)
        timed("swiglu_fwd", lambda: M.swiglu_fwd(gu), 3 * T * F * 2)
        timed("swiglu_bwd", lambda: M.swiglu_bwd(gu, do), 5 * T * F * 2)
    if only is None or "xent" in only:
        V = args.vocab
        logits = torch.randn(T, V, device=dev).to(bf)
        tgt = torch.randint(0, V, (T,), device=dev)
        timed("xent_fwd_bwd", lambda: M.xent_fwd_bwd_(logits, tgt, 1.0 / T), 2 * T * V * 2)
    if only is None or "comm" in only:
        world = 4
        n = 64 * 1024 * 1024                       # elements of the reduced shard (128 MB bf16)
        srcs = [torch.randn(n, device=dev).to(bf) for _ in range(world)]
        out = torch.empty(n, dtype=bf, device=dev)
        partials = torch.zeros(2048, dtype=torch.float32, device=dev)
        seg = (_ReduceSeg * 1)()
        seg[0].dst = out.data_ptr()
        for r in range(world):
            seg[0].src[r] = srcs[r].data_ptr()
        segs = torch.frombuffer(seg, dtype=torch.uint8).clone().to(dev)
        prefix = torch.tensor([0, n * 2 // 16], dtype=torch.int64, device=dev)
        for ctas in (148, 1184):
            timed("reduce_segments[4 sources, {} CTAs]".format(ctas),
                  lambda: ops().comm_reduce_segments(world, segs, 1, prefix, n * 2 // 16, 1.0 / world,
                                                     partials, ctas, 1),
                  (world + 1) * n * 2)
        gseg = (_GatherSeg * world)()
        gprefix = [0]
        chunk = n // world
        for r in range(world):
            gseg[r].src_off, gseg[r].dst_off, gseg[r].src_rank = 0, r * chunk * 2, r
            gprefix.append(gprefix[-1] + chunk * 2 // 16)
        gsegs = torch.frombuffer(gseg, dtype=torch.uint8).clone().to(dev)
        gpre = torch.tensor(gprefix, dtype=torch.int64, device=dev)
        bases = [s.data_ptr() for s in srcs]
        for ctas in (64, 296):
            timed("gather[4 segments, {} CTAs]".format(ctas),
                  lambda: ops().comm_gather(bases, gsegs, world, out, gpre, gprefix[-1], ctas),
                  2 * n * 2)


if __name__ == "__main__":
    main()
