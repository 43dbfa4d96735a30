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

OPTIMIZERS = ("gefen", "gefen_muon", "hybrid", "adamw")


@dataclass
class FindLRResult:
    lr: float
    method: str
    optimizer: str
    curve: List[Dict[str, float]] = field(default_factory=list)
    details: Dict[str, object] = field(default_factory=dict)


def build_optimizer(model: nn.Module, optimizer: str, lr: float, *, weight_decay: float = 0.0,
                    fused: bool = True, adjust_lr_fn: str = "match_rms_adamw"):
    """The requested optimizer family at ``lr`` (names of the reference tool, ``tools/find_lr.py:80-120``):
    ``gefen``; ``hybrid`` = GefenMuonHybrid over the whole model; ``gefen_muon`` = GefenMuon on the
    hidden 2-D matrices only (everything else stays frozen for the probe); ``adamw``."""
    from .. import Gefen, GefenMuon, GefenMuonHybrid

    if optimizer == "adamw":
        return torch.optim.AdamW(model.parameters(), lr=lr, weight_decay=weight_decay)
    use_fused = fused and all(p.is_cuda for p in model.parameters())
    if optimizer == "gefen":
        return Gefen([(n, p) for n, p in model.named_parameters() if p.requires_grad], lr=lr,
                     weight_decay=weight_decay, fused=use_fused)
    if optimizer == "hybrid":
        return GefenMuonHybrid(model, lr=lr, weight_decay=weight_decay, fused=use_fused,
                               adjust_lr_fn=adjust_lr_fn)
    if optimizer == "gefen_muon":
        from .run_model_calibration import split_params_for_muon

        muon, _ = split_params_for_muon(model)
        if not muon:
            raise ValueError("gefen_muon: model has no 2D hidden matrices to optimize")
        return GefenMuon(muon, lr=lr, weight_decay=weight_decay, fused=use_fused, adjust_lr_fn=adjust_lr_fn)
    raise ValueError("unknown optimizer {!r}; choose from {}".format(optimizer, OPTIMIZERS))


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


class _HFCausalLM(nn.Module):
    """A Hugging Face causal LM behind the ``(tokens, targets) -> loss`` call of the decoder presets."""

    def __init__(self, inner):
        super().__init__()
        self.inner = inner

    def forward(self, tokens, targets):
        full = torch.cat([tokens, targets[:, -1:]], dim=1)
        return self.inner(input_ids=full, labels=full).loss


class _HFModelFactory:
    """Picklable factory of a local Hugging Face checkpoint (workers are spawned)."""

    def __init__(self, path: str, dtype: str):
        self.path, self.dtype = path, dtype

    def __call__(self) -> nn.Module:
        from transformers import AutoModelForCausalLM

        inner = AutoModelForCausalLM.from_pretrained(self.path, dtype=getattr(torch, self.dtype),
                                                     low_cpu_mem_usage=True, local_files_only=True)
        inner.config.use_cache = False
        return _HFCausalLM(inner).train()


def _hf_blocks(model_path, dataset, split, seq, max_rows, eval_blocks):
    from types import SimpleNamespace

    from transformers import AutoTokenizer

    tok = AutoTokenizer.from_pretrained(model_path, local_files_only=True)
    return build_token_stream(tok, SimpleNamespace(dataset=dataset, split=split, seq=seq + 1, max_rows=max_rows,
                                                   eval_blocks=eval_blocks))


def find_lr_parallel_sweep(model_factory, train_blocks=None, eval_blocks=None, *, optimizer: str = "gefen",
                           sweep_lrs: Optional[List[float]] = None, devices: Optional[List[str]] = None,
                           sweep_steps: int = 80, warmup: int = 10, bs: int = 8, seed: int = 0,
                           weight_decay: float = 0.0, timeout_s: float = 3600.0, dtype: str = "bfloat16",
                           dataset: Optional[str] = None, split: str = "train", seq: int = 512,
                           max_rows: int = 0, fused: bool = True, adjust_lr_fn: str = "match_rms_adamw",
                           verbose: bool = True, worker_timeout: Optional[float] = None) -> FindLRResult:
    """The sweep of :func:`find_lr` with one spawned worker per device; a worker that fails
    reports its traceback through the queue and the whole call raises within ``timeout_s``.

    Two call forms: ``(model_factory, train_blocks, eval_blocks, ...)`` with token blocks in hand,
    or the reference tool's ``(model_path, devices, dataset=..., seq=..., eval_blocks=N, ...)``
    (``tools/find_lr.py:351-372``), which loads a local Hugging Face checkpoint in every worker and
    tokenises ``dataset`` (a local text / json / jsonl file, or an installed dataset name)."""
    import torch.multiprocessing as mp

    if isinstance(model_factory, str):
        model_path = model_factory
        if isinstance(train_blocks, (list, tuple)) and devices is None:
            devices = list(train_blocks)
        if dataset is None:
            raise ValueError("the model-path call form needs dataset=<file or installed dataset name>")
        n_eval = int(eval_blocks) if isinstance(eval_blocks, int) else 48
        train_blocks, eval_blocks = _hf_blocks(model_path, dataset, split, seq, max_rows, n_eval)
        model_factory = _HFModelFactory(model_path, dtype)
    if worker_timeout is not None:
        timeout_s = worker_timeout
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


def find_lr_sharded_sweep(model: str, train_blocks=None, *, world: Optional[int] = None,
                          sweep_lrs: Optional[List[float]] = None, sweep_steps: int = 40, warmup: int = 5,
                          bs: int = 1, seed: int = 0, weight_decay: float = 0.0, clip: Optional[float] = 1.0,
                          overrides: Optional[dict] = None, timeout_s: float = 3600.0,
                          devices: Optional[List[str]] = None, optimizer: str = "gefen", dtype: str = "bfloat16",
                          dataset: Optional[str] = None, split: str = "train", seq: int = 512, max_rows: int = 0,
                          eval_blocks: int = 48, fused: bool = True, adjust_lr_fn: str = "match_rms_adamw",
                          verbose: bool = True, worker_timeout: Optional[float] = None,
                          tokenizer: Optional[str] = None) -> FindLRResult:
    """lr sweep for a decoder preset sharded over ``world`` GPUs by ``ShardedTrainer``; the final
    training loss of the short run ranks the candidates.

    The reference tool's keywords (``tools/find_lr.py:550-571``) are accepted: ``devices`` (second
    positional or keyword) gives the world size, ``worker_timeout`` the time limit, and with
    ``dataset`` plus ``tokenizer`` (a local tokenizer folder) the token blocks are built here.
    ``model`` names a decoder preset: the sharded runtime owns its own model classes, it does not
    wrap Hugging Face modules; ``optimizer`` must be ``"gefen"``, ``dtype`` ``"bfloat16"``."""
    import torch.multiprocessing as mp

    if isinstance(train_blocks, (list, tuple)) and devices is None:        # (model, devices, ...)
        devices, train_blocks = list(train_blocks), None
    if devices is not None and world is None:
        world = len(devices)
    if worker_timeout is not None:
        timeout_s = worker_timeout
    if optimizer != "gefen" or dtype != "bfloat16":
        raise ValueError("the sharded sweep runs the fused Gefen update in bf16; got optimizer={!r}, "
                         "dtype={!r}".format(optimizer, dtype))
    if train_blocks is None:
        if dataset is None or tokenizer is None:
            raise ValueError("pass train_blocks, or dataset= and tokenizer= to build them")
        train_blocks, _ = _hf_blocks(tokenizer, dataset, split, seq, max_rows, eval_blocks)
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
def _row_text(row) -> str:
    """Text of one dataset row: a string, a ``text``-like field, or instruction / input / output."""
    if isinstance(row, str):
        return row
    if isinstance(row, dict):
        if row.get("instruction"):
            return "\n".join(x for x in (row.get("instruction", ""), row.get("input", ""), row.get("output", ""))
                             if x)
        for key in ("text", "content", "output", "completion", "body"):
            if row.get(key):
                return row[key]
    return ""


def _load_texts(dataset: str, split: str = "train", max_rows: int = 0) -> List[str]:
    """Texts of a local ``.txt`` / ``.json`` / ``.jsonl`` file, or of an installed Hugging Face
    dataset when ``dataset`` is not a path (no download is attempted beyond what ``datasets``
    finds in its cache)."""
    import json
    import os

    if os.path.exists(dataset):
        if dataset.endswith(".jsonl"):
            with open(dataset) as fh:
                texts = [_row_text(json.loads(line)) for line in fh if line.strip()]
        elif dataset.endswith(".json"):
            with open(dataset) as fh:
                loaded = json.load(fh)
            texts = [_row_text(r) for r in (loaded if isinstance(loaded, list) else [loaded])]
        else:
            with open(dataset) as fh:
                texts = [fh.read()]
    else:
        from datasets import load_dataset

        texts = [_row_text(r) for r in load_dataset(dataset, split=split)]
    texts = [t for t in texts if t]
    return texts[:max_rows] if max_rows and max_rows > 0 else texts


def build_token_stream(tok, args):
    """Tokenise ``args.dataset`` (fields ``dataset, split, max_rows, seq, eval_blocks``), pack the
    ids into ``[N, seq]`` blocks separated by EOS and hold out the last blocks for evaluation:
    ``(train_blocks, eval_blocks)`` (reference ``tools/find_lr.py:710-727``)."""
    seq = int(args.seq)
    eos = tok.eos_token_id if getattr(tok, "eos_token_id", None) is not None else 0
    ids: List[int] = []
    for text in _load_texts(args.dataset, getattr(args, "split", "train"), getattr(args, "max_rows", 0)):
        ids.extend(tok(text, add_special_tokens=False)["input_ids"])
        ids.append(eos)
    n_blocks = len(ids) // seq
    if n_blocks < 2:
        raise ValueError("only {} tokens -> {} blocks at seq={}; need >=2. Use a bigger dataset, a smaller "
                         "seq, or raise max_rows.".format(len(ids), n_blocks, seq))
    blocks = torch.tensor(ids[:n_blocks * seq], dtype=torch.long).view(n_blocks, seq)
    n_eval = max(1, min(int(getattr(args, "eval_blocks", 1)), n_blocks // 5))
    return blocks[:-n_eval], blocks[-n_eval:]


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
