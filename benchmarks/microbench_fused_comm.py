#!/usr/bin/env python
"""Fused compute + collective kernels against their rooflines, on N GPUs of one node.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29600 \
        benchmarks/microbench_fused_comm.py [--iters 10]

Builds a one-layer Llama-3-8B-shaped ``ShardedTrainer`` (so that the arenas, tables and flags are
the real ones), then times, with CUDA events and the maximum over ranks:

* the all-gather-fused QKV projection (``gemm_ag_bf16``: fetch CTAs pull the peers' q/k/v row
  shards while the tcgen05 tiles of the rows that have landed are computed), next to the same GEMM
  on weights that are already local and to "gather kernel, then GEMM";
* the reduce-scatter of one layer's gradients by peer loads (``reduce_segments_kernel``);
* the parameter all-gather of one layer by the copy engines and by the peer-load kernel.

Roofline of a fused kernel = the slower of FLOPs / measured cuBLAS bf16 throughput and bytes that
must cross NVLink / 770 GB/s (the measured peer-copy bandwidth per direction of these B200 systems).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

NVLINK_GBS = 770.0


def peak_tflops() -> float:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["bf16_tflops"])
    return 1590.0


def main():
    from gefen_x_b200.models.decoder import get_config
    from gefen_x_b200.ops import tcgemm
    from gefen_x_b200.ops._ext import ops
    from gefen_x_b200.parallel.fsdp import ShardedTrainer
    from gefen_x_b200.ops import update as U

    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--tokens", type=int, default=4096)
    args = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    cfg = get_config("llama3-8b", n_layers=1)
    tr = ShardedTrainer(cfg, device=dev, dtype=torch.bfloat16, world=world, rank=rank, lr=6e-6,
                        clip_grad_norm=1.0, seed=1, ag_gemm=True, gather_mode="kernel", reduce_mode="kernel")
    g = torch.Generator().manual_seed(rank)
    tok = torch.randint(0, cfg.vocab_size, (2, args.tokens // 2 + 1), generator=g).to(dev)
    for _ in range(2):                                   # builds every table, fills the gradient buffers
        tr.step(tok[:, :-1], tok[:, 1:])
    torch.cuda.synchronize()
    tr.check_status()
    peak = peak_tflops()
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)

    def timed(fn):
        ts = []
        for i in range(args.iters + 2):
            flush.fill_(i & 0xFF)
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if i >= 2:
                ts.append(e0.elapsed_time(e1))
        ts.sort()
        t = torch.tensor([ts[len(ts) // 2]], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def report(name, ms, flops=0.0, link_bytes=0.0, note=""):
        target = max(flops / (peak * 1e9), link_bytes / (NVLINK_GBS * 1e6))       # milliseconds
        rec = {"kernel": name, "ms": ms, "roofline_ms": target, "fraction_of_roofline": target / ms if ms else None,
               "tflops": flops / ms / 1e9 if flops else None,
               "link_gbs": link_bytes / ms / 1e6 if link_bytes else None, "n_gpus": world, "note": note}
        if rank == 0:
            print(json.dumps(rec), flush=True)

    grp = tr.groups[0]
    T, H = args.tokens, cfg.hidden
    n_rows = cfg.q_dim + 2 * cfg.kv_dim
    flat = tr.ring[0]
    h1 = torch.randn(T, H, device=dev).bfloat16()
    flops = 2.0 * T * n_rows * H
    remote = n_rows * H * 2 * (world - 1) / world
    fused = tr._qkv_fn(0, flat)
    ms_fused = timed(lambda: fused(h1))
    wqkv = flat[:n_rows * H].view(n_rows, H)
    ms_local = timed(lambda: tcgemm.gemm(h1, wqkv))
    qkv_specs = [sp for sp in grp.specs if sp.name.endswith(tr._QKV)]
    tab = tr._gather_table_for(grp, qkv_specs)

    def gather_then_gemm():
        ops().comm_gather(tr.arena.base_ptrs, tab[0], tab[1], flat, tab[2], tab[3], tr.gather_ctas)
        tcgemm.gemm(h1, wqkv)

    ms_seq = timed(gather_then_gemm)
    report("all-gather fused into the QKV GEMM (gemm_ag_bf16, {} fetch CTAs)".format(tr.ag_fetch_ctas),
           ms_fused, flops, remote,
           "tcgen05 GEMM alone on local weights: {:.3f} ms; gather kernel then GEMM: {:.3f} ms".format(ms_local, ms_seq))
    for n_fetch in (4, 8, 32):
        # the arrival counters are monotonic per launch: start a fresh series for another fetch width
        torch.cuda.synchronize()
        dist.barrier()
        tr._ag_count[0].zero_()
        tr._ag_flags[0].zero_()
        tr._ag_launches[0] = 0
        tr.ag_fetch_ctas = n_fetch
        f2 = tr._qkv_fn(0, flat)
        report("all-gather fused into the QKV GEMM (gemm_ag_bf16, {} fetch CTAs)".format(n_fetch),
               timed(lambda: f2(h1)), flops, remote)

    # reduce-scatter of the layer's gradients: peer loads, and in-switch reduction (multimem.ld_reduce on
    # the multicast mapping of the gradient buffers) where the arena has one.  Either way every GPU sends
    # (world - 1) slices of the size of a shard, which is the link roofline; the in-switch variant
    # receives one reduced shard instead of (world - 1) slices.
    partials = torch.zeros(2048, dtype=torch.float32, device=dev)
    was_nvls = tr.nvls
    for use_mc in ((False, True) if getattr(tr.arena, "mc_base", 0) else (False,)):
        tr.nvls = use_mc
        segs, n_segs, prefix, total, _copies = tr._build_reduce_table(grp, "all")
        own = total * 16
        for ctas in (148, 592):
            ms = timed(lambda: ops().comm_reduce_segments(world, segs, n_segs, prefix, total, 1.0 / world, partials,
                                                          ctas, U.DTYPE_CODE[torch.bfloat16], use_mc))
            name = "reduce-scatter by multimem.ld_reduce (reduce_segments_mc_kernel, {} CTAs)" if use_mc else \
                "reduce-scatter by peer loads (reduce_segments_kernel, {} CTAs)"
            report(name.format(ctas), ms, 0.0, own * (world - 1),
                   "shard of {:.0f} MB summed from {} ranks".format(own / 1e6, world))
    tr.nvls = was_nvls

    # parameter all-gather of the layer
    layer_bytes = grp.full_numel * 2
    for mode, lanes in (("kernel", 1), ("ce", 1), ("ce", 4), ("ce", 8)):
        tr.gather_mode = mode
        tr.copy_lanes = lanes
        ms = timed(lambda: tr._gather_into(grp, flat))
        report("parameter all-gather of one layer ({})".format(
                   "copy engines, {} stream(s)".format(lanes) if mode == "ce" else "gather_kernel, 64 CTAs"),
               ms, 0.0, layer_bytes * (world - 1) / world, "{:.0f} MB per layer".format(layer_bytes / 1e6))
    tr.check_status()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
