#!/usr/bin/env python
"""Flagship benchmark: sharded (FSDP2-style) full fine-tuning throughput with Gefen.

    python bench.py --gpus N --steps K --warmup W [--model qwen3-4b|llama3-8b] [--impl ours|reference]

Metric (the reference's headline, see its harness conventions at reference
``benchmarks/optimizer-sweep/sweep_cell.py:420-453`` and
``benchmarks/microbench/bench_muon_fsdp2.py:134-142``): training tokens per second
of the whole job (all GPUs), device-timed with CUDA events as the max over ranks,
plus the optimizer-step time and the optimizer-state bytes per parameter.
Default model: the Llama-3-8B shape (the headline configuration), two sequences of 2048
uniform-random tokens per GPU (one for qwen3-4b), weak scaling, random-init bf16 weights, Gefen with the factored second moment,
lr 6e-6, global-norm clipping at 1.0.  One JSON line is printed by rank 0.

For N > 1 launch with ``python -m torch.distributed.run --nproc-per-node N ...``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "fsdp2_full_ft_tokens_per_sec"
BATCH_PER_GPU = {"qwen3-4b": 1, "llama3-8b": 2}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama3-8b", choices=["llama3-8b", "qwen3-4b", "qwen3-1.7b", "qwen3-0.6b", "tiny-llama"])
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=0, help="sequences per GPU (0 = the config's)")
    ap.add_argument("--layers", type=int, default=0, help="debug only: override the layer count")
    ap.add_argument("--rs-mode", default=None)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--ag-gemm", action="store_true", help="all-gather fused into the QKV projection")
    ap.add_argument("--optimizer", default="gefen", choices=["gefen", "muon_hybrid"])
    ap.add_argument("--fp8-ns", action="store_true",
                    help="muon_hybrid: Newton-Schulz products in e4m3 (off by default: the benchmark dtype is bf16)")
    ap.add_argument("--gather", default="ce", choices=["ce", "kernel"],
                    help="parameter all-gather by copy engines or by a peer-load kernel")
    ap.add_argument("--reduce-ctas", type=int, default=148)
    ap.add_argument("--reduce", default="ce", choices=["ce", "kernel"],
                    help="gradient reduce-scatter: copy engines + local sum, or peer loads in the kernel")
    ap.add_argument("--attn", default="sdpa", choices=["sdpa", "tcgen05"],
                    help="attention: fused library kernel, or tcgen05 GEMMs + own row kernels")
    ap.add_argument("--nvls", default="auto", choices=["auto", "on", "off"],
                    help="gradient reduce-scatter through NVSwitch (multimem.ld_reduce); auto: off unless GEFENX_NVLS=1 "
                         "(measured slower on 2 GPUs, level on 8)")
    ap.add_argument("--copy-lanes", type=int, default=4,
                    help="auxiliary streams over which the copy-engine transfers of a gather / reduce are spread")
    ap.add_argument("--gemm-schedule", default="auto", choices=["auto", "static", "dynamic"],
                    help="tile schedule of the pair GEMM: fixed assignment, or tiles drawn from a device counter "
                         "(auto: dynamic with several ranks)")
    ap.add_argument("--gemm", default="tcgen05", choices=["tcgen05", "library"],
                    help="layer GEMMs: own tcgen05 kernels with fused epilogues (default), or the vendor library")
    ap.add_argument("--trace", action="store_true",
                    help="after the timed loops, print the per-phase device times of one more step (stderr)")
    return ap.parse_args()


def dist_setup(n_gpus: int):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != n_gpus:
        if world == 1 and n_gpus > 1:
            raise SystemExit("--gpus {} needs torch.distributed.run with --nproc-per-node {}".format(
                n_gpus, n_gpus))
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world, local


def provenance(dev) -> dict:
    """Where a number came from: code revision, library versions, device."""
    import subprocess

    def git(*a):
        try:
            return subprocess.run(["git", "-C", ROOT] + list(a), capture_output=True, text=True,
                                  timeout=10).stdout.strip()
        except Exception:
            return ""

    return {"git_commit": git("rev-parse", "--short", "HEAD") or None,
            "git_dirty": bool(git("status", "--porcelain")) if git("rev-parse", "--short", "HEAD") else None,
            "torch": torch.__version__, "cuda": torch.version.cuda,
            "gpu": torch.cuda.get_device_name(dev)}


def max_over_ranks(value: float, world: int) -> float:
    if world == 1:
        return value
    import torch.distributed as dist

    t = torch.tensor([value], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier_sync(world: int) -> None:
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
    torch.cuda.synchronize()


def timed_loop(step_fn, steps: int, world: int) -> float:
    """K steps between barrier+synchronize on both sides; CUDA-event milliseconds, max over ranks."""
    barrier_sync(world)
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        step_fn(i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    barrier_sync(world)
    return max_over_ranks(ms, world)


def run_ours(args):
    from gefen_x_b200.models.decoder import get_config
    from gefen_x_b200.ops import _ext
    from gefen_x_b200.parallel.fsdp import ShardedTrainer
    from gefen_x_b200.utils.clocks import ClockSampler

    rank, world, local = dist_setup(args.gpus)
    dev = torch.device("cuda", local)
    if args.attn != "sdpa":
        from gefen_x_b200.ops import model as _model_ops

        _model_ops.set_attention_impl(args.attn)
    from gefen_x_b200.ops import gemm as _gemm_ops

    _gemm_ops.set_backend(args.gemm)
    over = {"n_layers": args.layers} if args.layers else {}
    cfg = get_config(args.model, **over)
    B = args.batch or BATCH_PER_GPU.get(args.model, 1)
    S = args.seq_len
    trainer = ShardedTrainer(cfg, device=dev, dtype=torch.bfloat16, world=world, rank=rank,
                             lr=6e-6, clip_grad_norm=1.0, factored_v_2d=True, seed=1234,
                             rs_mode=args.rs_mode, ag_gemm=args.ag_gemm, optimizer=args.optimizer,
                             gather_mode=args.gather, reduce_ctas=args.reduce_ctas, reduce_mode=args.reduce,
                             nvls={"auto": None, "on": True, "off": False}[args.nvls],
                             gemm_schedule=args.gemm_schedule, copy_lanes=args.copy_lanes,
                             muon_kwargs=dict(ns_schedule="standard", ns_steps=5, fp8_ns=args.fp8_ns)
                             if args.optimizer == "muon_hybrid" else None)
    gen = torch.Generator().manual_seed(1000 + rank)
    n_batches = max(args.steps, 4)
    host_tok = [torch.randint(0, cfg.vocab_size, (B, S + 1), generator=gen).pin_memory()
                for _ in range(n_batches)]
    dev_tok = [t.to(dev) for t in host_tok]

    def dev_step(i):
        t = dev_tok[i % n_batches]
        return trainer.step(t[:, :-1], t[:, 1:])

    losses = []

    def e2e_step(i):
        t = host_tok[i % n_batches]
        loss = trainer.step(t[:, :-1], t[:, 1:])   # pinned host -> device inside step
        losses.append(float(loss.item()))          # device -> host read of the result

    for i in range(args.warmup):
        dev_step(i)
    trainer.check_status()

    # optimizer-step time: CUDA events around opt.step inside the timed steps
    opt_ms = []
    orig_step = trainer.opt.step
    orig_muon = trainer.muon.step if trainer.muon is not None else None

    def timed_opt_step(*a, **k):
        a0 = torch.cuda.Event(enable_timing=True)
        a1 = torch.cuda.Event(enable_timing=True)
        a0.record()
        r = orig_step(*a, **k)
        a1.record()
        opt_ms.append((a0, a1))
        return r

    trainer.opt.step = timed_opt_step
    if orig_muon is not None:
        def timed_muon_step(*a, **k):
            a0 = torch.cuda.Event(enable_timing=True)
            a1 = torch.cuda.Event(enable_timing=True)
            a0.record()
            r = orig_muon(*a, **k)
            a1.record()
            opt_ms.append((a0, a1))
            return r

        trainer.muon.step = timed_muon_step
    sampler = ClockSampler(gpu_index=local)
    if rank == 0:
        sampler.start()
    l0 = _ext.kernel_launches()
    ms = timed_loop(dev_step, args.steps, world)
    launches = _ext.kernel_launches() - l0
    clocks = sampler.stop() if rank == 0 else {}
    trainer.opt.step = orig_step
    if orig_muon is not None:
        trainer.muon.step = orig_muon
    opt_step_ms = max_over_ranks(sum(a.elapsed_time(b) for a, b in opt_ms) / max(1, args.steps), world)
    trainer.check_status()

    e2e = None
    if not args.no_e2e:
        e2e_ms = timed_loop(e2e_step, args.steps, world)
        tokens = world * B * S * args.steps
        e2e = {"value": tokens / (e2e_ms / 1e3), "unit": "tokens/s",
               "h2d_bytes_per_step": int(2 * B * S * 8), "d2h_bytes_per_step": 4,
               "ms_per_step": e2e_ms / args.steps, "last_loss": losses[-1] if losses else None}
    trainer.check_status()
    if args.trace:
        t = dev_tok[0]
        _, phases = trainer.traced_step(t[:, :-1], t[:, 1:])
        print("rank {} phases {}".format(rank, json.dumps({k: round(v, 2) for k, v in phases.items()})),
              file=sys.stderr, flush=True)
    tokens = world * B * S * args.steps
    peak_gib = max_over_ranks(torch.cuda.max_memory_allocated(dev) / 2 ** 30, world)
    out = {
        "metric": METRIC, "value": tokens / (ms / 1e3), "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 (Newton-Schulz products e4m3)" if (args.fp8_ns and args.optimizer == "muon_hybrid") else "bf16",
        "data": "synthetic uniform-random tokens, random-init N(0,0.02) weights",
        "impl": "ours",
        "opt_step_ms": opt_step_ms,
        "state_bytes_per_param": trainer.state_bytes_per_param(),
        "gpu_launches": int(launches),
        "peak_mem_gib": round(peak_gib, 2),
        "provenance": provenance(dev),
        "clocks": clocks,
        "e2e": e2e,
        "config": {"model": args.model, "layers": cfg.n_layers, "params": trainer.num_params(),
                   "global_batch": world * B, "seq_len": S,
                   "parallelism": "fsdp{}".format(world) if world > 1 else "single",
                   "optimizer": ("Gefen factored_v_2d lr6e-6 clip1.0" if args.optimizer == "gefen" else
                                 "GefenMuonHybrid (Muon NS-5 standard, quantized momentum; Gefen backup) "
                                 "lr6e-6 clip1.0"),
                   "l2": "working set per step (weights+grads, GBs) exceeds the 126 MB L2"},
        # how this implementation ran the config (kept out of `config`, which both arms share)
        "impl_config": {"rs_mode": trainer.rs_mode, "ag_gemm": trainer.ag_gemm, "attention": args.attn,
                        "gemm": args.gemm, "gather": trainer.gather_mode, "reduce": trainer.reduce_mode,
                        "reduce_ctas": trainer.reduce_ctas, "sparse_embedding": trainer.sparse_embed, "nvls": trainer.nvls,
                        "gemm_schedule": args.gemm_schedule, "copy_lanes": args.copy_lanes,
                        # kernel family of the optimizer's launch plans: 1 register-pipelined, 2 NVLS
                        # sources, 3 streamed through shared-memory rings, 0 generic
                        "update_plan_kinds": sorted({int(getattr(pl, "fast", -1)) for pl in
                                                     getattr(getattr(trainer.opt, "_plan_cache", None), "_plans", {}).values()})},
    }
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        from baseline.reference_arm import run_reference

        run_reference(args)
        return
    run_ours(args)


if __name__ == "__main__":
    main()
