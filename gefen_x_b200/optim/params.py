"""Parameter routing for the Muon hybrid: hidden 2-D matrices to Muon, the rest to the backup.

A parameter in both halves would be stepped twice and a trainable parameter in
neither would silently never train, so the split lives in one place and is
validated at construction.  Behaviour follows reference ``src/gefen/params.py``
(default substrings ``:30-37``, split ``:65-101``, validation ``:127-187``).
"""
from __future__ import annotations

import logging
from typing import Iterable, List, Tuple

import torch
import torch.nn as nn

logger = logging.getLogger(__name__)

# Case-insensitive name fragments that keep a 2-D weight out of Muon: token / position
# embeddings and output heads are vocabulary or class projections, not hidden matrices.
DEFAULT_BACKUP_SUBSTRINGS: Tuple[str, ...] = ("embed", "wte", "wpe", "lm_head", "classifier", "score")

Named = Tuple[str, nn.Parameter]


def is_muon_param(name: str, param, backup_substrings=DEFAULT_BACKUP_SUBSTRINGS) -> bool:
    if param.ndim != 2:
        return False
    low = name.lower()
    return not any(s.lower() in low for s in backup_substrings)


def _embedding_weight_ids(model: nn.Module) -> set:
    """ids of every ``nn.Embedding`` / ``nn.EmbeddingBag`` weight (catches tied heads by identity)."""
    out = set()
    for mod in model.modules():
        if isinstance(mod, (nn.Embedding, nn.EmbeddingBag)):
            w = getattr(mod, "weight", None)
            if w is not None:
                out.add(id(w))
    return out


def split_params_for_muon(model: nn.Module,
                          backup_substrings: Iterable[str] = DEFAULT_BACKUP_SUBSTRINGS
                          ) -> Tuple[List[Named], List[Named]]:
    """``(muon_named, backup_named)`` over the trainable parameters of ``model``."""
    subs = tuple(backup_substrings)
    emb = _embedding_weight_ids(model)
    muon: List[Named] = []
    backup: List[Named] = []
    for name, p in model.named_parameters():
        if not p.requires_grad:
            continue
        (muon if (id(p) not in emb and is_muon_param(name, p, subs)) else backup).append((name, p))
    logger.info("split_params_for_muon: %d muon / %d backup params; backup = %s",
                len(muon), len(backup), [n for n, _ in backup])
    return muon, backup


def split_named_for_muon(named: Iterable[Named],
                         backup_substrings: Iterable[str] = DEFAULT_BACKUP_SUBSTRINGS
                         ) -> Tuple[List[Named], List[Named]]:
    """Name-substring routing of an iterable of ``(name, param)`` pairs (no module information)."""
    subs = tuple(backup_substrings)
    muon, backup = [], []
    for name, p in named:
        if not getattr(p, "requires_grad", True):
            continue
        (muon if is_muon_param(name, p, subs) else backup).append((name, p))
    return muon, backup


def _check_pairs(items, which: str) -> None:
    for it in items:
        if (isinstance(it, (tuple, list)) and len(it) == 2 and isinstance(it[0], str)
                and isinstance(it[1], torch.Tensor)):
            continue
        raise TypeError(
            "validate_split expects the {} list to contain (name, param) pairs, got {!r}. Pass named "
            "parameters (e.g. model.named_parameters() or the lists from split_params_for_muon), or "
            "build the optimizer via GefenMuonHybrid.from_model(model, ...)".format(which, type(it)))


def validate_split(muon_named_params, backup_named_params, model: nn.Module = None):
    """Raise on a split that double-steps or drops a parameter; returns the two lists."""
    muon = list(muon_named_params)
    backup = list(backup_named_params)
    _check_pairs(muon, "muon")
    _check_pairs(backup, "backup")
    mids = {id(p) for _, p in muon}
    bids = {id(p) for _, p in backup}
    if len(mids) != len(muon):
        raise ValueError("Duplicate parameter object in the muon list")
    if len(bids) != len(backup):
        raise ValueError("Duplicate parameter object in the backup list")
    both = mids & bids
    if both:
        raise ValueError(
            "Parameter(s) {} appear in BOTH the muon and backup lists; they would be stepped twice "
            "per optimizer step".format([n for n, p in muon if id(p) in both]))
    names = [str(n).lower() for n, _ in muon] + [str(n).lower() for n, _ in backup]
    if len(set(names)) != len(names):
        seen, dup = set(), set()
        for n in names:
            (dup if n in seen else seen).add(n)
        raise ValueError(
            "Duplicate parameter name(s) {} across the muon/backup lists; the per-parameter state "
            "keys on the name, so duplicates collide".format(sorted(dup)))
    if model is not None:
        covered = mids | bids
        missing = [n for n, p in model.named_parameters() if p.requires_grad and id(p) not in covered]
        if missing:
            raise ValueError(
                "Trainable parameter(s) {} are in neither the muon nor backup list; they would "
                "never be optimized".format(missing))
    return muon, backup
