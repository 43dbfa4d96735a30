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
    return _build.load_cuda(required=required)


def ops():
    available(required=True)
    return torch.ops.gefenx
