"""Reference arm of ``bench.py``: the unmodified reference optimizer on its stock path.

Runs the reference package installed under ``baseline/_ref`` (``gefen.Gefen``,
its own JIT-built CUDA kernels) on a Hugging Face ``transformers`` model of the
benchmark's architecture with random-init bf16 weights, sharded with torch
FSDP2 ``fully_shard`` (one process per GPU over NCCL) exactly like the
reference's own FSDP2 harnesses (reference ``src/gefen/tools/find_lr.py:467-474``,
``benchmarks/sharding-sweep/fsdp2_convergence.py:196-201``,
``benchmarks/arch-compat/validate_fsdp.py:78-93``).  Nothing of this repository's
models, kernels or runtime is imported here.  Same metric, same timing rules and
same JSON line as the other arm.
"""
from __future__ import annotations

import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")

MODELS = {
    "qwen3-4b": dict(kind="qwen3", vocab_size=151936, hidden_size=2560, num_hidden_layers=36,
                     num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                     intermediate_size=9728, rope_theta=1e6, tie_word_embeddings=True,
                     rms_norm_eps=1e-6),
    "llama3-8b": dict(kind="llama", vocab_size=128256, hidden_size=4096, num_hidden_layers=32,
                      num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                      intermediate_size=14336, rope_theta=5e5, tie_word_embeddings=False,
                      rms_norm_eps=1e-5),
}
BATCH_PER_GPU = {"qwen3-4b": 1, "llama3-8b": 2}


def _unavailable(why: str) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)


def run_reference(args) -> None:
    if not os.path.isdir(os.path.join(REF, "gefen")):
        _unavailable("baseline/_ref is missing: the reference was not installed on this box")
        return
    try:
        _run(args)
    except Exception as exc:  # report instead of crashing the driver's run
        import traceback

        traceback.print_exc()
        _unavailable("{}: {}".format(type(exc).__name__, str(exc).splitlines()[0][:200]))


def _run(args) -> None:
    import torch

    sys.path.insert(0, REF)
    os.environ.setdefault("GEFEN_KERNEL_BUILD_ROOT", os.path.join(HERE, "_ref_build"))
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    import gefen  # the reference package
    from transformers import AutoModelForCausalLM, LlamaConfig, Qwen3Config

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit("--gpus {} needs torch.distributed.run --nproc-per-node {}".format(
            args.gpus, args.gpus))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    import torch.distributed as dist

    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    spec = dict(MODELS[args.model])
    kind = spec.pop("kind")
    if args.layers:
        spec["num_hidden_layers"] = args.layers
    S = args.seq_len
    B = args.batch or BATCH_PER_GPU.get(args.model, 1)
    spec["max_position_embeddings"] = max(S, 4096)
    cfg = (Qwen3Config if kind == "qwen3" else LlamaConfig)(**spec)
    cfg._attn_implementation = "sdpa"
    torch.manual_seed(1234)
    with torch.device(dev):
        model = AutoModelForCausalLM.from_config(cfg, torch_dtype=torch.bfloat16)
    model.train()
    model.config.use_cache = False
    n_params = sum(p.numel() for p in model.parameters())
    if world > 1:
        from torch.distributed.fsdp import fully_shard

        for layer in model.model.layers:
            fully_shard(layer)
        fully_shard(model)
    if getattr(args, "optimizer", "gefen") == "muon_hybrid":
        opt = gefen.GefenMuonHybrid(model, lr=6e-6, ns_schedule="standard", ns_steps=5,
                                    sharded_mode="distributed" if world > 1 else "exact")
    else:
        opt = gefen.Gefen(list(model.named_parameters()), lr=6e-6, factored_v_2d=True)

    gen = torch.Generator().manual_seed(1000 + rank)
    n_batches = max(args.steps, 4)
    host_tok = [torch.randint(0, spec["vocab_size"], (B, S), generator=gen).pin_memory()
                for _ in range(n_batches)]
    dev_tok = [t.to(dev) for t in host_tok]
    opt_events = []

    def one_step(tok, time_opt=False):
        loss = model(input_ids=tok, labels=tok).loss
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        if time_opt:
            a0 = torch.cuda.Event(enable_timing=True)
            a1 = torch.cuda.Event(enable_timing=True)
            a0.record()
            opt.step()
            a1.record()
            opt_events.append((a0, a1))
        else:
            opt.step()
        opt.zero_grad(set_to_none=True)
        return loss

    def barrier_sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(fn):
        barrier_sync()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.steps):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        barrier_sync()
        return max_ranks(ms)

    for i in range(args.warmup):
        one_step(dev_tok[i % n_batches])
    clocks = {}
    sampler = None
    if rank == 0:
        try:
            sys.path.insert(0, os.path.dirname(HERE))
            from gefen_x_b200.utils.clocks import ClockSampler  # read-only nvidia-smi poller

            sampler = ClockSampler(gpu_index=local)
            sampler.start()
        except Exception:
            sampler = None
    ms = timed(lambda i: one_step(dev_tok[i % n_batches], time_opt=True))
    if sampler is not None:
        clocks = sampler.stop()
    opt_ms = max_ranks(sum(a.elapsed_time(b) for a, b in opt_events) / max(1, len(opt_events)))
    losses = []

    def e2e(i):
        tok = host_tok[i % n_batches].to(dev, non_blocking=True)
        losses.append(float(one_step(tok).item()))

    e2e_ms = timed(e2e)
    state_bytes = 0
    own = 0
    children = [c for c in (getattr(opt, "muon", None), getattr(opt, "backup", None)) if c is not None] or [opt]
    for child in children:
        for p, st in child.state.items():
            for v in st.values():
                if torch.is_tensor(v):
                    state_bytes += v.numel() * v.element_size()
    for p in model.parameters():
        pl = p.to_local() if hasattr(p, "to_local") else p
        own += pl.numel()
    tokens = world * B * S * args.steps
    out = {
        "metric": "fsdp2_full_ft_tokens_per_sec", "value": tokens / (ms / 1e3), "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic uniform-random tokens, random-init weights", "impl": "reference",
        "opt_step_ms": opt_ms, "state_bytes_per_param": state_bytes / max(1, own),
        "clocks": clocks,
        "e2e": {"value": tokens / (e2e_ms / 1e3), "unit": "tokens/s",
                "h2d_bytes_per_step": int(B * S * 8), "d2h_bytes_per_step": 4,
                "ms_per_step": e2e_ms / args.steps, "last_loss": losses[-1] if losses else None},
        "config": {"model": args.model, "layers": spec["num_hidden_layers"], "params": n_params,
                   "global_batch": world * B, "seq_len": S,
                   "parallelism": "fsdp{}".format(world) if world > 1 else "single",
                   "optimizer": ("Gefen factored_v_2d lr6e-6 clip1.0"
                                 if getattr(args, "optimizer", "gefen") == "gefen" else
                                 "GefenMuonHybrid (Muon NS-5 standard, quantized momentum; Gefen backup) "
                                 "lr6e-6 clip1.0"),
                   "l2": "working set per step (weights+grads, GBs) exceeds the 126 MB L2"},
        # how this arm ran the config (kept out of `config`, which both arms share)
        "impl_config": {"optimizer_class": "reference gefen.{}".format(type(opt).__name__),
                        "model_impl": "transformers {} sdpa".format(kind),
                        "sharding": "torch fully_shard" if world > 1 else "none"},
    }
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()
