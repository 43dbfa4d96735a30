"""Access to the compiled sm_100a operators (``torch.ops.gefenx``)."""
from __future__ import annotations

import torch

from .. import build as _build

DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def available(required: bool = False) -> bool:
    """Whether the extension is loaded (loading it on first call).

    ``required=True`` raises with the build/load error instead of returning
    False; the CUDA code paths use it so that a missing extension on a GPU box
    is loud rather than a silent fall back to torch ops.
    """
    ok = _build.load_cuda(required=required)
    if ok:
        from . import _fake

        _fake.register()
    return ok


# kernels launched by one call of each operator (for launch accounting)
_KERNELS_PER_CALL = {"factored_update": 4, "muon_epilogue": 3, "desc_size": 0, "rmsnorm_bwd_partials": 0}
launch_count = 0


class _CountingOps:
    """``torch.ops.gefenx`` with a running count of the kernels it launched."""

    def __init__(self, ns):
        self._ns = ns
        self._cache = {}

    def __getattr__(self, name):
        fn = self._cache.get(name)
        if fn is None:
            raw = getattr(self._ns, name)
            n = _KERNELS_PER_CALL.get(name, 1)

            def fn(*a, _raw=raw, _n=n, **k):
                global launch_count
                launch_count += _n
                return _raw(*a, **k)

            self._cache[name] = fn
        return fn


_proxy = None


def ops():
    global _proxy
    if _proxy is None:
        available(required=True)
        _proxy = _CountingOps(torch.ops.gefenx)
    return _proxy


def kernel_launches() -> int:
    """Number of this package's kernels launched so far in this process."""
    return launch_count
