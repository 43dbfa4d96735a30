"""Run the lr probes of ``lr_calibration`` on a decoder preset (or a Hugging Face model).

    python -m gefen_x_b200.tools.run_model_calibration --model tiny-llama --optimizer gefen_muon

Counterpart of the reference's HF-model runner (``src/gefen/tools/run_model_calibration.py:106-259``);
``--hf PATH`` loads a local ``transformers`` checkpoint instead of a preset (no network access
is attempted).
"""
from __future__ import annotations

import argparse
import json
import sys

import torch

from .find_lr import _closure_from_blocks, build_optimizer
from .lr_calibration import calibrate_relative, calibrate_vs_adamw, measure_update_rms


def load_model(args, device, dtype):
    if args.hf:
        from transformers import AutoModelForCausalLM

        model = AutoModelForCausalLM.from_pretrained(args.hf, torch_dtype=dtype, local_files_only=True)
        inner = model.to(device)

        class Wrapper(torch.nn.Module):
            def __init__(self):
                super().__init__()
                self.inner = inner

            def forward(self, tokens, targets):
                return self.inner(input_ids=tokens, labels=tokens).loss

        return Wrapper(), inner.config.vocab_size
    from ..models.decoder import DecoderLM, get_config

    cfg = get_config(args.model)
    return DecoderLM(cfg, device=device, dtype=dtype, seed=args.seed), cfg.vocab_size


def run_one(args):
    device = torch.device(args.device or ("cuda" if torch.cuda.is_available() else "cpu"))
    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    model, vocab = load_model(args, device, dtype)
    g = torch.Generator().manual_seed(args.seed)
    blocks = torch.randint(0, vocab, (args.num_blocks, args.seq_len + 1), generator=g)
    closure = _closure_from_blocks(model, blocks, device, args.bs, args.seed)
    opt = build_optimizer(model, args.optimizer, args.lr, fused=device.type == "cuda")
    out = {}
    stats = measure_update_rms(opt, closure, num_steps=args.steps, warmup=args.warmup)
    out["update_rms"] = [s.__dict__ for s in stats]
    rel = calibrate_relative(opt, closure, num_steps=args.steps, warmup=args.warmup)
    out["relative"] = {"reference": rel.reference_label, "multipliers": rel.multipliers}
    if args.vs_adamw:
        out["vs_adamw"] = [p.__dict__ for p in calibrate_vs_adamw(opt, closure, num_steps=args.steps,
                                                                  warmup=args.warmup)]
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="tiny-llama")
    ap.add_argument("--hf", default=None)
    ap.add_argument("--optimizer", default="gefen", choices=["gefen", "gefen_muon", "adamw"])
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--steps", type=int, default=12)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--bs", type=int, default=4)
    ap.add_argument("--seq-len", type=int, default=64)
    ap.add_argument("--num-blocks", type=int, default=32)
    ap.add_argument("--vs-adamw", action="store_true")
    ap.add_argument("--device", default=None)
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args(argv)
    print(json.dumps(run_one(args), default=str))
    return 0


if __name__ == "__main__":
    sys.exit(main())
