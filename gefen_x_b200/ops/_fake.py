"""Meta ("fake") implementations of the ``gefenx::`` operators for ``torch.compile``.

Every kernel operator writes its results into tensors the caller passes (declared ``Tensor(a!)`` in
the schema) and returns nothing, so its fake implementation is empty: tracing only needs to know
that the call is legal on fake tensors.  ``period_errors`` is the one operator that returns a
tensor.  Operators that write through raw device addresses (descriptor tables, peer pointers)
declare no tensor mutation the tracer could see; they are marked as having side effects so that a
compiled graph can neither drop nor reorder them.  The optimizers' ``step`` itself is excluded from
tracing (``torch.compiler.disable``): it runs its launch plans eagerly inside a compiled training
step, and CUDA-graph capture of the step goes through ``capturable=True``.

The reference registers its kernels as custom ops with fake implementations for the same purpose
(reference ``src/gefen/kernels/automatic_gefen_fused.py:449-509``, ``:554-572``;
``src/gefen/kernels/period_variance.py:36-59``).
"""
from __future__ import annotations

import torch

_VOID_OPS = (
    "block_update", "factored_update", "reduce_sources", "clip_coef", "histogram", "remap_indices",
    "quantize_rows_e4m3", "quantize_cols_e4m3_t", "dequantize", "gemm_bf16", "gemm_pair_bf16", "gemm_pair_e4m3", "gemm_ag_bf16", "muon_epilogue",
    "comm_wait", "comm_gather", "comm_scatter_apply", "comm_reduce_segments", "comm_gather_rows",
    "comm_scatter_add_rows", "comm_allreduce_scalar", "rmsnorm_fwd", "rmsnorm_bwd", "rope",
    "flash_attention_fwd", "attn_softmax", "attn_row_dot", "attn_bwd_rows", "swiglu_fwd", "swiglu_bwd",
    "xent_fwd_bwd",
)
# write through addresses held in byte tables / integer lists: invisible to the tracer
_HIDDEN_WRITES = ("block_update", "factored_update", "reduce_sources", "comm_wait", "comm_scatter_apply",
                  "comm_reduce_segments", "comm_allreduce_scalar", "comm_signal", "comm_copy_list")
_registered = False


def register() -> None:
    """Register the fake implementations once the extension library is loaded (idempotent)."""
    global _registered
    if _registered:
        return
    _registered = True
    lib = torch.library

    def _nothing(*args, **kwargs):
        return None

    for name in _VOID_OPS:
        if hasattr(torch.ops.gefenx, name):
            try:
                lib.register_fake("gefenx::" + name, _nothing)
            except RuntimeError:          # already registered (module reloaded)
                pass

    def _period_errors(flat, divisors, input_is_squared):
        return flat.new_empty((divisors.numel(), 296), dtype=torch.float64)

    try:
        lib.register_fake("gefenx::period_errors", _period_errors)
    except RuntimeError:
        pass
    try:
        from torch.fx.node import has_side_effect

        for name in _HIDDEN_WRITES:
            op = getattr(torch.ops.gefenx, name, None)
            if op is not None:
                has_side_effect(op.default)
    except Exception:                     # pragma: no cover - fx internals moved
        pass
