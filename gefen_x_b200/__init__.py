"""gefen_x_b200 – Blackwell-native (sm_100a) memory-efficient optimizer framework.

Public names are resolved lazily so that ``import gefen_x_b200`` stays cheap and
never triggers a native build (same façade idea as the reference's
``src/gefen/__init__.py:10-59``).
"""
from __future__ import annotations

import importlib

__version__ = "0.1.0"

_EXPORTS = {
    "Gefen": ".optim.gefen",
    "GefenMuon": ".optim.muon",
    "GefenMuonHybrid": ".optim.hybrid",
    "split_params_for_muon": ".optim.params",
    "validate_split": ".optim.params",
    "DEFAULT_BACKUP_SUBSTRINGS": ".optim.params",
    "GefenDCPState": ".ckpt.dcp",
    "GefenSavePlanner": ".ckpt.dcp",
    "GefenFileSystemWriter": ".ckpt.dcp",
    "find_period_by_block_variance": ".quant.partitioning",
    "exact_dp": ".quant.codebook",
    "ShardedTrainer": ".parallel.fsdp",
    "DecoderLM": ".models.decoder",
    "ModelConfig": ".models.decoder",
}

# submodules reachable as attributes; ``kernels`` is the name the reference gives its kernel
# wrappers (``src/gefen/__init__.py:52-58``), here the ``ops`` package
_SUBMODULES = {"kernels": ".ops", "ops": ".ops", "params": ".optim.params"}

__all__ = sorted(_EXPORTS) + ["kernels", "__version__"]


def __getattr__(name):
    sub = _SUBMODULES.get(name)
    if sub is not None:
        value = importlib.import_module(sub, __name__)
        globals()[name] = value
        return value
    mod = _EXPORTS.get(name)
    if mod is None:
        raise AttributeError("module 'gefen_x_b200' has no attribute {!r}".format(name))
    value = getattr(importlib.import_module(mod, __name__), name)
    globals()[name] = value
    return value


def __dir__():
    return __all__
