"""Learning-rate finder for Gefen / GefenMuonHybrid / AdamW.

* :func:`find_lr` – range test (exponential ramp) or a short-fine-tune sweep on one device;
* :func:`find_lr_parallel_sweep` – the sweep with the candidate lrs spread over several GPUs
  (one spawned process per device);
* :func:`find_lr_sharded_sweep` – the sweep on a model too large for one GPU: every candidate
  runs sharded over all ranks through :class:`~gefen_x_b200.parallel.fsdp.ShardedTrainer`;
* ``python -m gefen_x_b200.tools.find_lr`` – command line on the built-in decoder presets with
  a token file (``--tokens file.pt``, a ``[N, seq]`` int64 tensor) or synthetic tokens.

Same entry points as the reference (``src/gefen/tools/find_lr.py``: ``find_lr`` ``:166-254``,
``find_lr_parallel_sweep`` ``:351-443``, ``find_lr_sharded_sweep`` ``:550-660``, ``main``
``:799-889``); the sharded sweep uses this package's runtime instead of torch ``fully_shard``.
"""
from __future__ import annotations

import argparse
import json
import math
import socket
import sys
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Union

import torch
import torch.nn as nn

from .lr_calibration import lr_range_test

OPTIMIZERS = ("gefen", "gefen_muon", "adamw")


@dataclass
class FindLRResult:
    lr: float
    method: str
    optimizer: str
    curve: List[Dict[str, float]] = field(default_factory=list)
    details: Dict[str, object] = field(default_factory=dict)


def build_optimizer(model: nn.Module, optimizer: str, lr: float, *, weight_decay: float = 0.0,
                    fused: bool = True, adjust_lr_fn: str = "match_rms_adamw"):
    from .. import Gefen, GefenMuonHybrid

    use_fused = fused and all(p.is_cuda for p in model.parameters())
    if optimizer == "gefen":
        return Gefen(model.named_parameters(), lr=lr, weight_decay=weight_decay, fused=use_fused)
    if optimizer == "gefen_muon":
        return GefenMuonHybrid(model, lr=lr, weight_decay=weight_decay, fused=use_fused,
                               adjust_lr_fn=adjust_lr_fn)
    if optimizer == "adamw":
        return torch.optim.AdamW(model.parameters(), lr=lr, weight_decay=weight_decay)
    raise ValueError("optimizer must be one of {}".format(OPTIMIZERS))


def _model_loss(model, tokens):
    out = model(tokens[:, :-1], tokens[:, 1:])
    return out.loss if hasattr(out, "loss") else out


def _closure_from_blocks(model, blocks: torch.Tensor, device, bs: int, seed: int):
    gen = torch.Generator().manual_seed(seed)
    n = blocks.shape[0]

    def closure():
        idx = torch.randint(0, n, (bs,), generator=gen)
        loss = _model_loss(model, blocks[idx].to(device))
        loss.backward()
        return loss.detach()

    return closure


@torch.no_grad()
def _eval_loss(model, eval_blocks: torch.Tensor, device, bs: int) -> float:
    was = model.training
    model.eval()
    total, count = 0.0, 0
    for i in range(0, eval_blocks.shape[0], bs):
        t = eval_blocks[i:i + bs].to(device)
        total += float(_model_loss(model, t)) * t.shape[0]
        count += t.shape[0]
    model.train(was)
    return total / max(1, count)


def _snapshot(model):
    return {k: v.detach().clone() for k, v in model.state_dict().items()}


def _short_finetune(model, train_blocks, optimizer, device, *, steps, warmup, bs, seed) -> float:
    closure = _closure_from_blocks(model, train_blocks, device, bs, seed)
    base = [float(g["lr"]) for g in optimizer.param_groups]
    last = float("nan")
    for it in range(steps):
        scale = min(1.0, (it + 1) / max(1, warmup))
        for g, b in zip(optimizer.param_groups, base):
            g["lr"] = b * scale
        optimizer.zero_grad()
        last = float(closure())
        optimizer.step()
        if not math.isfinite(last):
            break
    return last


def find_lr(model, train_data: Union[torch.Tensor, Callable[[], torch.Tensor]], *, optimizer: str = "gefen",
            method: str = "range_test", eval_blocks: Optional[torch.Tensor] = None,
            device: Optional[Union[str, torch.device]] = None, weight_decay: float = 0.0,
            fused: bool = True, adjust_lr_fn: str = "match_rms_adamw", restore: bool = True,
            num_iter: int = 100, start_lr: float = 1e-6, end_lr: float = 1e-1, smooth_beta: float = 0.9,
            diverge_factor: float = 5.0, sweep_lrs: Optional[List[float]] = None, sweep_steps: int = 80,
            warmup: int = 10, bs: int = 8, seed: int = 0, verbose: bool = True) -> FindLRResult:
    """Recommend a base lr for ``optimizer`` on ``model`` with a few batches.

    ``train_data`` is a ``[N, seq]`` int64 tensor of token blocks or a ready closure (forward +
    backward, returns the loss).  ``method="sweep"`` needs ``eval_blocks``.
    """
    if optimizer not in OPTIMIZERS:
        raise ValueError("optimizer must be one of {}".format(OPTIMIZERS))
    if method not in ("range_test", "sweep"):
        raise ValueError("method must be 'range_test' or 'sweep'")
    device = torch.device(device) if device is not None else next(model.parameters()).device
    saved = _snapshot(model) if restore else None
    try:
        if method == "range_test":
            closure = train_data if callable(train_data) else _closure_from_blocks(
                model, train_data, device, bs, seed)
            opt = build_optimizer(model, optimizer, start_lr, weight_decay=weight_decay, fused=fused,
                                  adjust_lr_fn=adjust_lr_fn)
            res = lr_range_test(opt, closure, start_lr=start_lr, end_lr=end_lr, num_iter=num_iter,
                                smooth_beta=smooth_beta, diverge_factor=diverge_factor, restore=False)
            curve = [{"lr": a, "loss": b, "smoothed": c} for a, b, c in zip(res.lrs, res.losses, res.smoothed)]
            if verbose:
                print("range test: suggested lr {:.3e} (min-loss lr {:.3e}, diverged at {})".format(
                    res.suggested_lr, res.min_loss_lr, res.diverged_at))
            return FindLRResult(res.suggested_lr, method, optimizer, curve,
                                {"min_loss_lr": res.min_loss_lr, "diverged_at": res.diverged_at})
        if eval_blocks is None or callable(train_data):
            raise ValueError("method='sweep' needs token blocks for train_data and eval_blocks")
        lrs = list(sweep_lrs) if sweep_lrs else [1e-5, 3e-5, 1e-4, 3e-4, 1e-3, 3e-3]
        start = _snapshot(model)
        curve = []
        for lr in lrs:
            model.load_state_dict(start)
            opt = build_optimizer(model, optimizer, lr, weight_decay=weight_decay, fused=fused,
                                  adjust_lr_fn=adjust_lr_fn)
            train_loss = _short_finetune(model, train_data, opt, device, steps=sweep_steps, warmup=warmup,
                                         bs=bs, seed=seed)
            ev = _eval_loss(model, eval_blocks, device, bs) if math.isfinite(train_loss) else float("inf")
            curve.append({"lr": lr, "train_loss": train_loss, "eval_loss": ev})
            if verbose:
                print("sweep lr {:.3e}: train {:.4f} eval {:.4f}".format(lr, train_loss, ev))
        best = min(curve, key=lambda r: r["eval_loss"])
        return FindLRResult(best["lr"], method, optimizer, curve, {})
    finally:
        if saved is not None:
            model.load_state_dict(saved)


# ---------------------------------------------------------------- multi-GPU sweep
def distribute_lrs(lrs: List[float], devices: List[str]) -> Dict[str, List[float]]:
    """Round-robin assignment of the candidates to devices."""
    out = {d: [] for d in devices}
    for i, lr in enumerate(lrs):
        out[devices[i % len(devices)]].append(lr)
    return out


def _sweep_worker(device: str, lr_list: List[float], cfg: dict, q) -> None:
    try:
        torch.manual_seed(cfg["seed"])
        model = cfg["model_factory"]().to(device)
        res = find_lr(model, cfg["train_blocks"], optimizer=cfg["optimizer"], method="sweep",
                      eval_blocks=cfg["eval_blocks"], device=device, sweep_lrs=lr_list,
                      sweep_steps=cfg["sweep_steps"], warmup=cfg["warmup"], bs=cfg["bs"],
                      seed=cfg["seed"], weight_decay=cfg["weight_decay"], verbose=False, restore=False)
        q.put(("OK", device, res.curve))
    except Exception:  # noqa: BLE001
        import traceback

        q.put(("ERROR", device, traceback.format_exc()))


def find_lr_parallel_sweep(model_factory: Callable[[], nn.Module], train_blocks: torch.Tensor,
                           eval_blocks: torch.Tensor, *, optimizer: str = "gefen",
                           sweep_lrs: Optional[List[float]] = None, devices: Optional[List[str]] = None,
                           sweep_steps: int = 80, warmup: int = 10, bs: int = 8, seed: int = 0,
                           weight_decay: float = 0.0, timeout_s: float = 3600.0) -> FindLRResult:
    """The sweep of :func:`find_lr` with one spawned worker per device; a worker that fails
    reports its traceback through the queue and the whole call raises within ``timeout_s``."""
    import torch.multiprocessing as mp

    lrs = list(sweep_lrs) if sweep_lrs else [1e-5, 3e-5, 1e-4, 3e-4, 1e-3, 3e-3]
    if devices is None:
        n = torch.cuda.device_count()
        devices = ["cuda:{}".format(i) for i in range(n)] if n else ["cpu"]
    plan = {d: l for d, l in distribute_lrs(lrs, devices).items() if l}
    cfg = dict(model_factory=model_factory, train_blocks=train_blocks, eval_blocks=eval_blocks,
               optimizer=optimizer, sweep_steps=sweep_steps, warmup=warmup, bs=bs, seed=seed,
               weight_decay=weight_decay)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_sweep_worker, args=(d, l, cfg, q)) for d, l in plan.items()]
    for p in procs:
        p.start()
    curve, deadline, err = [], time.time() + timeout_s, None
    try:
        for _ in procs:
            tag, dev, payload = q.get(timeout=max(1.0, deadline - time.time()))
            if tag == "ERROR":
                err = "worker on {} failed:\n{}".format(dev, payload)
                break
            curve.extend(payload)
    finally:
        for p in procs:
            p.join(timeout=5 if err else max(1.0, deadline - time.time()))
            if p.is_alive():
                p.terminate()
    if err:
        raise RuntimeError(err)
    curve.sort(key=lambda r: r["lr"])
    best = min(curve, key=lambda r: r["eval_loss"])
    return FindLRResult(best["lr"], "sweep", optimizer, curve, {"devices": list(plan)})


# ---------------------------------------------------------------- sharded sweep
def _free_port() -> str:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return str(port)


def _shard_worker(rank: int, world: int, lr: float, cfg: dict, port: str, q) -> None:
    import os

    import torch.distributed as dist

    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = port
        cuda = torch.cuda.is_available()
        if cuda:
            torch.cuda.set_device(rank)
        if world > 1:
            dist.init_process_group("nccl" if cuda else "gloo", rank=rank, world_size=world)
        from ..models.decoder import get_config
        from ..parallel.fsdp import ShardedTrainer

        mcfg = get_config(cfg["model"], **cfg.get("overrides", {}))
        dev = torch.device("cuda", rank) if cuda else torch.device("cpu")
        tr = ShardedTrainer(mcfg, device=dev, dtype=torch.bfloat16 if cuda else torch.float32,
                            world=world, rank=rank, lr=lr, weight_decay=cfg["weight_decay"],
                            clip_grad_norm=cfg["clip"], seed=cfg["seed"])
        blocks = cfg["train_blocks"]
        gen = torch.Generator().manual_seed(cfg["seed"] + rank)
        last = float("nan")
        for it in range(cfg["sweep_steps"]):
            for g in tr.opt.param_groups:
                g["lr"] = lr * min(1.0, (it + 1) / max(1, cfg["warmup"]))
            idx = torch.randint(0, blocks.shape[0], (cfg["bs"],), generator=gen)
            t = blocks[idx]
            last = float(tr.step(t[:, :-1], t[:, 1:]).item())
            if not math.isfinite(last):
                break
        tr.check_status() if cuda else None
        if rank == 0:
            q.put(("OK", lr, last))
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
    except Exception:  # noqa: BLE001
        import traceback

        q.put(("ERROR", lr, traceback.format_exc()))


def find_lr_sharded_sweep(model: str, train_blocks: torch.Tensor, *, world: Optional[int] = None,
                          sweep_lrs: Optional[List[float]] = None, sweep_steps: int = 40, warmup: int = 5,
                          bs: int = 1, seed: int = 0, weight_decay: float = 0.0, clip: Optional[float] = 1.0,
                          overrides: Optional[dict] = None, timeout_s: float = 3600.0) -> FindLRResult:
    """lr sweep for a decoder preset sharded over ``world`` GPUs; the final training loss of the
    short run ranks the candidates."""
    import torch.multiprocessing as mp

    world = world or max(1, torch.cuda.device_count())
    lrs = list(sweep_lrs) if sweep_lrs else [1e-6, 3e-6, 1e-5, 3e-5, 1e-4]
    cfg = dict(model=model, train_blocks=train_blocks, sweep_steps=sweep_steps, warmup=warmup, bs=bs,
               seed=seed, weight_decay=weight_decay, clip=clip, overrides=overrides or {})
    ctx = mp.get_context("spawn")
    curve = []
    for lr in lrs:
        q = ctx.Queue()
        port = _free_port()
        procs = [ctx.Process(target=_shard_worker, args=(r, world, lr, cfg, port, q)) for r in range(world)]
        for p in procs:
            p.start()
        try:
            tag, _lr, payload = q.get(timeout=timeout_s)
        finally:
            for p in procs:
                p.join(timeout=60)
                if p.is_alive():
                    p.terminate()
        if tag == "ERROR":
            raise RuntimeError("sharded sweep at lr {} failed:\n{}".format(lr, payload))
        curve.append({"lr": lr, "train_loss": payload})
    finite = [r for r in curve if math.isfinite(r["train_loss"])]
    best = min(finite or curve, key=lambda r: r["train_loss"])
    return FindLRResult(best["lr"], "sharded_sweep", "gefen", curve, {"world": world})


# ---------------------------------------------------------------- command line
def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description="Learning-rate finder for the Gefen optimizers")
    ap.add_argument("--model", default="tiny-llama", help="decoder preset (models.decoder.PRESETS)")
    ap.add_argument("--optimizer", default="gefen", choices=OPTIMIZERS)
    ap.add_argument("--method", default="range_test", choices=["range_test", "sweep", "sharded_sweep"])
    ap.add_argument("--tokens", default=None, help="torch file with a [N, seq] int64 tensor of token blocks")
    ap.add_argument("--seq-len", type=int, default=128)
    ap.add_argument("--num-blocks", type=int, default=64)
    ap.add_argument("--bs", type=int, default=4)
    ap.add_argument("--num-iter", type=int, default=60)
    ap.add_argument("--start-lr", type=float, default=1e-6)
    ap.add_argument("--end-lr", type=float, default=1e-1)
    ap.add_argument("--sweep-lrs", type=float, nargs="*", default=None)
    ap.add_argument("--sweep-steps", type=int, default=40)
    ap.add_argument("--device", default=None)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--json", action="store_true")
    args = ap.parse_args(argv)

    from ..models.decoder import DecoderLM, get_config

    cfg = get_config(args.model)
    if args.tokens:
        blocks = torch.load(args.tokens)
    else:
        g = torch.Generator().manual_seed(args.seed)
        blocks = torch.randint(0, cfg.vocab_size, (args.num_blocks, args.seq_len + 1), generator=g)
    n_eval = max(1, blocks.shape[0] // 8)
    train, ev = blocks[n_eval:], blocks[:n_eval]
    if args.method == "sharded_sweep":
        res = find_lr_sharded_sweep(args.model, train, sweep_lrs=args.sweep_lrs,
                                    sweep_steps=args.sweep_steps, bs=args.bs, seed=args.seed)
    else:
        device = torch.device(args.device or ("cuda" if torch.cuda.is_available() else "cpu"))
        dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
        model = DecoderLM(cfg, device=device, dtype=dtype, seed=args.seed)
        res = find_lr(model, train, optimizer=args.optimizer, method=args.method, eval_blocks=ev,
                      device=device, num_iter=args.num_iter, start_lr=args.start_lr, end_lr=args.end_lr,
                      sweep_lrs=args.sweep_lrs, sweep_steps=args.sweep_steps, bs=args.bs, seed=args.seed,
                      verbose=not args.json)
    if args.json:
        print(json.dumps({"lr": res.lr, "method": res.method, "optimizer": res.optimizer,
                          "curve": res.curve}))
    else:
        print("recommended lr: {:.3e}".format(res.lr))
    return 0


if __name__ == "__main__":
    sys.exit(main())
