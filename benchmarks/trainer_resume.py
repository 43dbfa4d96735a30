#!/usr/bin/env python
"""Exact-resume gate for the optimizers inside a training loop.

For every recipe the same short run is made twice on a fixed token stream: once without
interruption, and once stopped at ``--split-step``, written to disk (model, optimizer, LR scheduler,
step and data position with ``torch.save``), reloaded into freshly constructed objects and continued.
The gate passes when the SHA-256 digests of the final model, optimizer and scheduler states of the
two runs are equal: a resumed run is then indistinguishable from one that never stopped, with
gradient accumulation and a warm-up schedule in play.

The loop is plain torch (the same contract a framework trainer relies on: ``state_dict`` /
``load_state_dict`` of model, optimizer and scheduler).  The reference has the same gate built on the
Hugging Face ``Trainer`` (reference ``benchmarks/trainer_resume/run.py``,
``tests/test_transformers_trainer_resume.py``); that trainer needs the ``accelerate`` package, which
this environment does not have.

    python benchmarks/trainer_resume.py --output-dir /tmp/resume --device cpu --steps 6 --split-step 2
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import struct
import sys
from typing import Any, Dict, Tuple

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

RECIPES = ("gefen", "gefen_block", "gefen_muon_hybrid")


# ---------------------------------------------------------------------------------------------
# digests
# ---------------------------------------------------------------------------------------------
def _feed(h, obj: Any) -> None:
    """Structural, order-independent for mappings, exact for tensors (dtype, shape, bytes)."""
    if torch.is_tensor(obj):
        t = obj.detach().cpu().contiguous()
        h.update(b"T" + str(t.dtype).encode() + str(tuple(t.shape)).encode())
        h.update(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
    elif isinstance(obj, dict):
        h.update(b"D%d" % len(obj))
        for k in sorted(obj, key=lambda x: (str(type(x)), str(x))):
            _feed(h, k)
            _feed(h, obj[k])
    elif isinstance(obj, (list, tuple)):
        h.update(b"L%d" % len(obj))
        for v in obj:
            _feed(h, v)
    elif isinstance(obj, bool) or obj is None:
        h.update(b"B" + repr(obj).encode())
    elif isinstance(obj, int):
        h.update(b"I" + str(obj).encode())
    elif isinstance(obj, float):
        h.update(b"F" + struct.pack("<d", obj))
    else:
        h.update(b"S" + str(obj).encode())


def state_digest(obj: Any) -> str:
    h = hashlib.sha256()
    _feed(h, obj)
    return h.hexdigest()


# ---------------------------------------------------------------------------------------------
# data and model
# ---------------------------------------------------------------------------------------------
class FixedTokenDataset(torch.utils.data.Dataset):
    """``samples`` rows of ``seq_len`` tokens drawn once from ``seed``; labels equal the inputs."""

    def __init__(self, samples: int, seq_len: int, vocab_size: int, seed: int):
        g = torch.Generator().manual_seed(seed)
        self.input_ids = torch.randint(0, vocab_size, (samples, seq_len), generator=g)

    def __len__(self) -> int:
        return self.input_ids.shape[0]

    def __getitem__(self, i: int) -> Dict[str, torch.Tensor]:
        row = self.input_ids[i]
        return {"input_ids": row, "labels": row, "attention_mask": torch.ones_like(row)}


def build_model(args, device, dtype):
    from gefen_x_b200.models.decoder import DecoderLM, get_config

    torch.manual_seed(args.seed)
    cfg = get_config("tiny-llama", n_layers=2, hidden=64, ffn=128, vocab_size=args.vocab_size)
    return DecoderLM(cfg, device=device, dtype=dtype, impl="torch" if device.type == "cpu" else "auto")


def build_optimizer(recipe: str, model, args):
    from gefen_x_b200 import Gefen, GefenMuonHybrid

    fused = not args.no_fused
    if recipe == "gefen":
        return Gefen(list(model.named_parameters()), lr=args.lr, weight_decay=0.01, fused=fused)
    if recipe == "gefen_block":
        return Gefen(list(model.named_parameters()), lr=args.lr, weight_decay=0.01, fused=fused,
                     factored_v_2d=False)
    if recipe == "gefen_muon_hybrid":
        return GefenMuonHybrid(model, lr=args.lr, weight_decay=0.01, ns_steps=args.ns_steps)
    raise ValueError("unknown recipe {!r}".format(recipe))


def build_scheduler(opt, args):
    warm = max(1, args.warmup_steps)
    return torch.optim.lr_scheduler.LambdaLR(opt, lambda s: min(1.0, (s + 1) / warm) * (1.0 - 0.5 * s / max(1, args.steps)))


# ---------------------------------------------------------------------------------------------
# the loop
# ---------------------------------------------------------------------------------------------
def _micro_batches(ds: FixedTokenDataset, args, start: int):
    """Deterministic order: sample index advances by one per micro-batch row, wrapping around."""
    pos = start
    while True:
        rows = [(pos + j) % len(ds) for j in range(args.batch_size)]
        pos += args.batch_size
        yield pos, torch.stack([ds[i]["input_ids"] for i in rows])


def train(recipe: str, args, out_dir: str, *, stop_at: int = 0, resume_from: str = "") -> Tuple[Any, Any, Any, Dict]:
    device = torch.device(args.device)
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[args.dtype]
    ds = FixedTokenDataset(args.samples, args.seq_len, args.vocab_size, args.seed + 1)
    model = build_model(args, device, dtype)
    opt = build_optimizer(recipe, model, args)
    sched = build_scheduler(opt, args)
    step, data_pos, losses = 0, 0, []
    if resume_from:
        ck = torch.load(os.path.join(resume_from, "checkpoint.pt"), map_location=device, weights_only=False)
        model.load_state_dict(ck["model"])
        opt.load_state_dict(ck["optimizer"])
        sched.load_state_dict(ck["scheduler"])
        step, data_pos, losses = ck["step"], ck["data_pos"], list(ck["losses"])
    batches = _micro_batches(ds, args, data_pos)
    last = stop_at or args.steps
    while step < last:
        total = 0.0
        for _ in range(args.gradient_accumulation_steps):
            data_pos, tok = next(batches)
            tok = tok.to(device)
            loss = model(tok[:, :-1], tok[:, 1:]) / args.gradient_accumulation_steps
            loss.backward()
            total += float(loss.detach())
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        sched.step()
        opt.zero_grad(set_to_none=True)
        step += 1
        losses.append(total)
    if stop_at:
        os.makedirs(out_dir, exist_ok=True)
        torch.save({"model": model.state_dict(), "optimizer": opt.state_dict(), "scheduler": sched.state_dict(),
                    "step": step, "data_pos": data_pos, "losses": losses}, os.path.join(out_dir, "checkpoint.pt"))
    return model, opt, sched, {"losses": losses, "step": step}


def _digests(model, opt, sched) -> Dict[str, str]:
    return {"model_sha256": state_digest(model.state_dict()),
            "optimizer_sha256": state_digest(opt.state_dict()),
            "scheduler_sha256": state_digest(sched.state_dict())}


def run(args) -> Dict[str, Any]:
    if not 0 < args.split_step < args.steps:
        raise ValueError("--split-step must lie strictly between 0 and --steps")
    summary: Dict[str, Any] = {"recipes": {}, "passed": True}
    for recipe in args.recipes:
        base_dir = os.path.join(args.output_dir, recipe)
        m, o, s, info = train(recipe, args, base_dir)
        baseline = dict(_digests(m, o, s), losses=info["losses"])
        train(recipe, args, base_dir, stop_at=args.split_step)
        m, o, s, info = train(recipe, args, base_dir, resume_from=base_dir)
        resumed = dict(_digests(m, o, s), losses=info["losses"])
        ok = all(baseline[k] == resumed[k] for k in ("model_sha256", "optimizer_sha256", "scheduler_sha256"))
        summary["recipes"][recipe] = {"baseline": baseline, "resumed": resumed, "passed": ok}
        summary["passed"] = summary["passed"] and ok
    return summary


# ---------------------------------------------------------------------------------------------
# command line
# ---------------------------------------------------------------------------------------------
def _recipe_list(text: str) -> Tuple[str, ...]:
    names = tuple(t.strip() for t in text.split(",") if t.strip())
    unknown = [n for n in names if n not in RECIPES]
    if unknown:
        raise argparse.ArgumentTypeError("unknown recipes: {} (known: {})".format(", ".join(unknown), ", ".join(RECIPES)))
    if len(set(names)) != len(names):
        raise argparse.ArgumentTypeError("duplicates in the recipe list")
    return names


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--output-dir", required=True)
    ap.add_argument("--recipes", type=_recipe_list, default=RECIPES)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--dtype", default="float32", choices=["float32", "bfloat16"])
    ap.add_argument("--no-fused", action="store_true", help="decomposed torch path even on CUDA")
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--split-step", type=int, default=2)
    ap.add_argument("--warmup-steps", type=int, default=2)
    ap.add_argument("--batch-size", type=int, default=2)
    ap.add_argument("--gradient-accumulation-steps", type=int, default=2)
    ap.add_argument("--seq-len", type=int, default=32)
    ap.add_argument("--samples", type=int, default=16)
    ap.add_argument("--vocab-size", type=int, default=256)
    ap.add_argument("--ns-steps", type=int, default=5)
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--seed", type=int, default=0)
    return ap.parse_args(argv)


def main() -> int:
    args = parse_args()
    summary = run(args)
    print(json.dumps(summary))
    return 0 if summary["passed"] else 1


if __name__ == "__main__":
    sys.exit(main())
