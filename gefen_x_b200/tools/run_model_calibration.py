"""Run the lr probes of ``lr_calibration`` on a decoder preset (or a Hugging Face model).

    python -m gefen_x_b200.tools.run_model_calibration --model tiny-llama --optimizer hybrid

Counterpart of the reference's HF-model runner (``src/gefen/tools/run_model_calibration.py:106-259``);
``--hf PATH`` loads a local ``transformers`` checkpoint instead of a preset (no network access
is attempted).
"""
from __future__ import annotations

import argparse
import itertools
import json
import math
import statistics
import sys
from collections import defaultdict

import torch

from .find_lr import _closure_from_blocks, build_optimizer
from .lr_calibration import calibrate_relative, calibrate_vs_adamw, measure_update_rms

_PROJECTIONS = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj", "qkv_proj",
                "gate_up_proj")
_NOT_HIDDEN = ("embed", "wte", "lm_head", "patch", "vision", "visual", "multi_modal", "mm_", "projector")

# Short texts of different kinds, cycled one per step so that the probe does not memorise one batch.
CORPUS = [
    "Block-wise quantised momentum keeps one byte per element and one magnitude per block of a parameter.",
    "The ferry left the harbour at dawn, and by noon the island was only a grey line behind the spray.",
    "for row in table:\n    total += row.price * row.count\nprint(round(total, 2))\n",
    "Either party may end this agreement with thirty days of written notice to the other party.",
    "Whisk the eggs with the milk, pour over the bread, and bake until the custard has just set.",
    "Ribosomes read the messenger RNA three bases at a time and add one amino acid for each codon.",
    "Operating income fell four percent as freight costs rose faster than the company could reprice.",
    "He sanded the plank along the grain, wiped off the dust, and brushed on the first thin coat of oil.",
]


def classify_param_type(name) -> str:
    """Coarse type of a parameter from its name: a projection name, embed, lm_head, norm, bias or
    other (same classes as the reference's ``tools/run_model_calibration.py:40-57``)."""
    n = (name or "").lower()
    for t in _PROJECTIONS:
        if t in n:
            return t
    if "embed" in n or "wte" in n:
        return "embed"
    if "lm_head" in n:
        return "lm_head"
    if "norm" in n or "layernorm" in n or ".ln" in n:
        return "norm"
    if "bias" in n:
        return "bias"
    return "other"


param_type = classify_param_type


def split_params_for_muon(model):
    """(hidden 2-D matrices, everything else) as named lists; embeddings, heads and vision /
    projector towers stay with the backup optimizer."""
    muon, backup = [], []
    for name, p in model.named_parameters():
        if not p.requires_grad:
            continue
        hidden = p.ndim == 2 and not any(k in name.lower() for k in _NOT_HIDDEN)
        (muon if hidden else backup).append((name, p))
    return muon, backup


def make_corpus_closure(model, tok, device, seq):
    """A closure over ``CORPUS``: each call runs forward + backward on the next text."""
    batches = []
    for text in CORPUS:
        enc = tok(text, return_tensors="pt", truncation=True, max_length=seq)
        mask = enc.get("attention_mask")
        batches.append((enc["input_ids"].to(device), None if mask is None else mask.to(device)))
    cyc = itertools.cycle(batches)

    def closure():
        ids, mask = next(cyc)
        out = model(input_ids=ids, attention_mask=mask, labels=ids)
        out.loss.backward()
        return out.loss.detach()

    return closure


def _summ(xs):
    xs = [x for x in xs if math.isfinite(x)]
    return (statistics.median(xs), min(xs), max(xs), len(xs)) if xs else None


def _load_hf(path, device, dtype):
    """(tokenizer, model) of a local Hugging Face checkpoint, in training mode (no network)."""
    from transformers import AutoModelForCausalLM, AutoTokenizer

    tok = AutoTokenizer.from_pretrained(path, local_files_only=True)
    model = AutoModelForCausalLM.from_pretrained(path, dtype=dtype, low_cpu_mem_usage=True, local_files_only=True)
    model.to(device)
    model.train()
    model.config.use_cache = False
    if hasattr(model, "gradient_checkpointing_enable"):
        model.gradient_checkpointing_enable()
    return tok, model


def run_hf_model(path, device, dtype, steps, warmup, seq, reference="adamw"):
    """The reference's per-model report: hybrid optimizer on a local HF checkpoint, per-type table
    of the AdamW / optimizer update-RMS ratio and the empirical Muon ``k`` (``match_rms_adamw``
    assumes 0.2); ``reference="self"`` prints the relative calibration instead."""
    from ..optim.hybrid import GefenMuonHybrid

    dev = torch.device(device)
    tok, model = _load_hf(path, dev, dtype)
    muon, backup = split_params_for_muon(model)
    print("MODEL {}: {} muon matrices, {} backup params".format(path, len(muon), len(backup)))
    opt = GefenMuonHybrid(muon, backup, lr=1e-3, weight_decay=0.1, fused=dev.type == "cuda", adjust_lr_fn=None)
    closure = make_corpus_closure(model, tok, dev, seq)
    result = {"model": str(path).rstrip("/").split("/")[-1]}
    if reference != "adamw":
        print(calibrate_relative(opt, closure, reference="gefen", num_steps=steps, warmup=warmup).summary())
        return result
    ratio_by_type, k_by_type, muon_k, backup_ratio = defaultdict(list), defaultdict(list), [], []
    for r in calibrate_vs_adamw(opt, closure, num_steps=steps, warmup=warmup):
        t = param_type(r.name)
        ratio_by_type[t].append(r.ratio)
        if r.is_muon and r.sqrt_max:
            k = r.active_ratio * r.ratio / r.sqrt_max
            k_by_type[t].append(k)
            muon_k.append(k)
        elif not r.is_muon:
            backup_ratio.append(r.ratio)
    print("  {:<14}{:<7}{:>4}{:>11}{:>11}".format("type", "kind", "n", "ratio med", "k_eff med"))
    for t in sorted(ratio_by_type):
        s = _summ(ratio_by_type[t])
        if s is None:
            continue
        ks = _summ(k_by_type[t]) if k_by_type[t] else None
        print("  {:<14}{:<7}{:>4}{:>11.3f}{:>11}".format(t, "muon" if ks else "backup", s[3], s[0],
                                                       "{:.3f}".format(ks[0]) if ks else "-"))
    result["muon_k"], result["backup_ratio"] = _summ(muon_k), _summ(backup_ratio)
    return result


def load_model(args, device, dtype):
    if isinstance(args, str):                       # the reference's call form: load_model(path, device, dtype)
        return _load_hf(args, torch.device(device), dtype)
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


def run_one(args, device=None, dtype=None, steps=40, warmup=5, seq=128, reference="adamw"):
    if isinstance(args, str):                       # the reference's call form: run_one(path, device, dtype, ...)
        return run_hf_model(args, device, dtype, steps, warmup, seq, reference)
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
    ap.add_argument("--optimizer", default="gefen", choices=["gefen", "gefen_muon", "hybrid", "adamw"])
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--steps", type=int, default=12)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--bs", type=int, default=4)
    ap.add_argument("--seq-len", type=int, default=64)
    ap.add_argument("--num-blocks", type=int, default=32)
    ap.add_argument("--vs-adamw", action="store_true")
    ap.add_argument("--device", default=None)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--models", nargs="+", default=None,
                    help="local Hugging Face checkpoints: per-model, per-parameter-type report (the reference's mode)")
    ap.add_argument("--dtype", default="bfloat16")
    ap.add_argument("--seq", type=int, default=128)
    ap.add_argument("--reference", choices=["adamw", "self"], default="adamw")
    args = ap.parse_args(argv)
    if args.models:
        device = args.device or ("cuda:0" if torch.cuda.is_available() else "cpu")
        results = [run_hf_model(path, device, getattr(torch, args.dtype), args.steps, args.warmup, args.seq,
                                args.reference) for path in args.models]
        print(json.dumps(results, default=str))
        return 0
    print(json.dumps(run_one(args), default=str))
    return 0


if __name__ == "__main__":
    sys.exit(main())
