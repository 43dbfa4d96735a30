"""Python entry points of the model kernels, each with a plain torch statement.

The torch statement is the fp32 oracle of the tests and the path taken by CPU
tensors; CUDA tensors go to ``csrc/model_ops.cu``.  The reference expresses
these with torch ops inside its benchmark model (reference
``benchmarks/training_matrix/tiny_qwen.py:113-138``, ``:180-181``, ``:250-259``).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from ._ext import available, ops

_KERNEL_DTYPES = (torch.float32, torch.bfloat16, torch.float16)


def _use_kernel(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype in _KERNEL_DTYPES and available(required=True)


# ---------------------------------------------------------------- RMSNorm
def rmsnorm_ref(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    rstd = torch.rsqrt(xf.square().mean(-1, keepdim=True) + eps)
    return (xf * rstd * w.float()).to(x.dtype)


def rmsnorm_fwd(x: torch.Tensor, w: torch.Tensor, eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """``y = x * rsqrt(mean(x^2) + eps) * w`` over the last dim; returns (y, rstd)."""
    d = x.shape[-1]
    if _use_kernel(x) and d % 8 == 0:
        x = x.contiguous()
        y = torch.empty_like(x)
        rstd = torch.empty(x.numel() // d, dtype=torch.float32, device=x.device)
        ops().rmsnorm_fwd(x, w.contiguous(), y, rstd, float(eps))
        return y, rstd
    xf = x.float()
    rstd = torch.rsqrt(xf.square().mean(-1, keepdim=True) + eps)
    return (xf * rstd * w.float()).to(x.dtype), rstd.reshape(-1)


def rmsnorm_bwd(dy: torch.Tensor, x: torch.Tensor, w: torch.Tensor, rstd: torch.Tensor,
                res: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns ``(dx, dw)`` with ``dw`` in fp32.  ``res`` (optional, shaped like ``x``) is added to
    ``dx`` inside the kernel: the gradient that reaches ``x`` along the residual path."""
    d = x.shape[-1]
    rows = x.numel() // d
    if _use_kernel(x) and d % 8 == 0 and d <= 16384:
        dy = dy.contiguous()
        x = x.contiguous()
        dx = torch.empty_like(x)
        npart = int(ops().rmsnorm_bwd_partials(rows, d))
        part = torch.empty(npart, d, dtype=torch.float32, device=x.device)
        dw = torch.empty(d, dtype=torch.float32, device=x.device)
        ops().rmsnorm_bwd(dy, x, w.contiguous(), rstd, dx, part, None if res is None else res.contiguous(), dw)
        return dx, dw
    xf, dyf, wf = x.float().reshape(rows, d), dy.float().reshape(rows, d), w.float()
    r = rstd.reshape(rows, 1)
    g = dyf * wf
    dx = r * (g - xf * (r * r) * (g * xf).sum(-1, keepdim=True) / d)
    if res is not None:
        dx = dx + res.float().reshape(rows, d)
    dw = (dyf * xf * r).sum(0)
    return dx.reshape(x.shape).to(x.dtype), dw


# ---------------------------------------------------------------- RoPE
def rope_tables(seq_len: int, head_dim: int, theta: float, device) -> Tuple[torch.Tensor, torch.Tensor]:
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim))
    ang = torch.outer(torch.arange(seq_len, dtype=torch.float64), inv)
    return ang.cos().float().to(device), ang.sin().float().to(device)


def rope_ref(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, inverse: bool = False,
             interleaved: bool = False) -> torch.Tensor:
    """x: [B, S, n, hd]; half-rotation (HF) or interleaved-pair layout."""
    s = sin if not inverse else -sin
    c = cos[None, :, None, :]
    s = s[None, :, None, :]
    xf = x.float()
    if interleaved:
        a, b = xf[..., 0::2], xf[..., 1::2]
        out = torch.stack((a * c - b * s, b * c + a * s), dim=-1).flatten(-2)
    else:
        h = x.shape[-1] // 2
        a, b = xf[..., :h], xf[..., h:]
        out = torch.cat((a * c - b * s, b * c + a * s), dim=-1)
    return out.to(x.dtype)


def rope_(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, inverse: bool = False,
          interleaved: bool = False) -> torch.Tensor:
    """In-place rotary embedding of a contiguous [B, S, n, hd] tensor."""
    if _use_kernel(x) and x.is_contiguous():
        B, S, n, hd = x.shape
        x2 = x.view(B * S, n * hd)
        ops().rope(x2, x2, cos, sin, S, n, hd, bool(inverse), bool(interleaved))
        return x
    x.copy_(rope_ref(x, cos, sin, inverse, interleaved))
    return x


def rope_into(dst2d: torch.Tensor, src2d: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, seq_len: int,
              n_heads: int, head_dim: int, inverse: bool = False, interleaved: bool = False) -> torch.Tensor:
    """``dst2d = rope(src2d)`` for ``[tokens, n_heads * head_dim]`` views whose rows may be strided
    (column slices of a fused projection buffer): rotation and (un)packing in one pass."""
    if _use_kernel(src2d) and src2d.stride(1) == 1 and dst2d.stride(1) == 1:
        ops().rope(dst2d, src2d, cos, sin, int(seq_len), int(n_heads), int(head_dim), bool(inverse),
                   bool(interleaved))
        return dst2d
    T = src2d.shape[0]
    x = src2d.reshape(T // seq_len, seq_len, n_heads, head_dim)
    dst2d.copy_(rope_ref(x, cos, sin, inverse, interleaved).reshape(T, n_heads * head_dim))
    return dst2d


# ---------------------------------------------------------------- SwiGLU
def swiglu_fwd(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` for ``gate_up = [gate | up]`` along the last dim."""
    f = gate_up.shape[-1] // 2
    if _use_kernel(gate_up) and f % 8 == 0:
        gate_up = gate_up.contiguous()
        out = torch.empty(*gate_up.shape[:-1], f, dtype=gate_up.dtype, device=gate_up.device)
        ops().swiglu_fwd(gate_up, out)
        return out
    g, u = gate_up[..., :f].float(), gate_up[..., f:].float()
    return (F.silu(g) * u).to(gate_up.dtype)


def swiglu_bwd(gate_up: torch.Tensor, dout: torch.Tensor) -> torch.Tensor:
    f = gate_up.shape[-1] // 2
    if _use_kernel(gate_up) and f % 8 == 0:
        gate_up = gate_up.contiguous()
        dgu = torch.empty_like(gate_up)
        ops().swiglu_bwd(gate_up, dout.contiguous(), dgu)
        return dgu
    g, u, dz = gate_up[..., :f].float(), gate_up[..., f:].float(), dout.float()
    sg = torch.sigmoid(g)
    dg = dz * u * sg * (1 + g * (1 - sg))
    du = dz * g * sg
    return torch.cat((dg, du), dim=-1).to(gate_up.dtype)


# ---------------------------------------------------------------- cross-entropy
def xent_fwd_bwd_(logits: torch.Tensor, targets: torch.Tensor, grad_scale: float,
                  ignore_index: int = -100) -> torch.Tensor:
    """Per-row loss; ``logits`` is overwritten with ``(softmax - onehot) * grad_scale``."""
    v = logits.shape[-1]
    rows = logits.numel() // v
    if _use_kernel(logits) and logits.is_contiguous():
        loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
        ops().xent_fwd_bwd(logits, targets.reshape(-1).contiguous(), loss, float(grad_scale),
                           int(ignore_index))
        return loss
    lf = logits.float().reshape(rows, v)
    t = targets.reshape(-1)
    valid = (t != ignore_index)
    lse = torch.logsumexp(lf, dim=-1)
    tc = t.clamp(min=0)
    loss = torch.where(valid, lse - lf.gather(1, tc[:, None]).squeeze(1), torch.zeros_like(lse))
    prob = torch.softmax(lf, dim=-1)
    prob[torch.arange(rows, device=lf.device), tc] -= 1.0
    prob = prob * (valid[:, None].float() * grad_scale)
    logits.copy_(prob.reshape(logits.shape).to(logits.dtype))
    return loss


# ---------------------------------------------------------------- attention
_ATTN_IMPL = "sdpa"


def set_attention_impl(name: str) -> None:
    """``"sdpa"``: the fused library kernel (default); ``"tcgen05"``: the tcgen05 GEMM plus own row
    kernels of :mod:`gefen_x_b200.ops.attention` (bf16 CUDA tensors; others fall back to sdpa)."""
    global _ATTN_IMPL
    if name not in ("sdpa", "tcgen05"):
        raise ValueError("attention implementation must be 'sdpa' or 'tcgen05'")
    _ATTN_IMPL = name


def attention_impl() -> str:
    return _ATTN_IMPL


def attention_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor):
    """Causal GQA attention on [B, S, n, hd] tensors.

    Returns ``(out [B, S, nq, hd], ctx)``; ``ctx`` feeds :func:`attention_bwd`.
    """
    if _ATTN_IMPL == "tcgen05":
        from . import attention as _att

        if _att.supported(q, k):
            out, ctx = _att.attention_fwd(q, k, v)
            return out, ("tcgen05", ctx)
    with torch.enable_grad():
        ql = q.detach().requires_grad_(True)
        kl = k.detach().requires_grad_(True)
        vl = v.detach().requires_grad_(True)
        groups = ql.shape[2] // kl.shape[2]
        o = F.scaled_dot_product_attention(
            ql.transpose(1, 2), kl.transpose(1, 2), vl.transpose(1, 2), is_causal=True,
            enable_gqa=groups > 1)
        o = o.transpose(1, 2)
    return o.detach(), (ql, kl, vl, o)


def attention_bwd(ctx, dout: torch.Tensor):
    if len(ctx) == 2 and isinstance(ctx[0], str):
        from . import attention as _att

        return _att.attention_bwd(ctx[1], dout)
    ql, kl, vl, o = ctx
    return torch.autograd.grad(o, (ql, kl, vl), dout)
