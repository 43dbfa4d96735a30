"""Llama / Qwen3-style decoder-only language model.

The reference contains no model code in its package; its only model is the
benchmark-only ``benchmarks/training_matrix/tiny_qwen.py`` (RMSNorm ``:113-123``,
RoPE ``:126-138``, GQA attention ``:141-171``, SwiGLU ``:174-181``, LM head + loss
``:250-259``).  This module supplies the model family named by the benchmark
configs (Llama-3-8B, Qwen3-4B, the 2-layer CPU config) in two forms that share
weights and math:

* a plain torch forward (autograd does the backward): CPU, fp32/fp64, and the
  numerical oracle of the tests;
* a layer-wise manual forward/backward built on the kernels of ``ops.model``
  and ``ops.gemm``: each decoder layer is one ``torch.autograd.Function`` and the
  sharded runtime (``parallel.fsdp``) drives the same layer functions directly,
  gathering a layer's weights before it runs and reducing its gradients after.

Weights of a layer live in one flat buffer: ``[q|k|v]`` and ``[gate|up]`` are
adjacent, so the projections run as single fused GEMMs while the optimizer still
sees HF-style individual matrices (``q_proj.weight`` ...) as row slices.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import gemm as G
from ..ops import model as M


@dataclass
class ModelConfig:
    vocab_size: int = 1024
    hidden: int = 256
    n_layers: int = 2
    n_heads: int = 4
    n_kv_heads: int = 2
    head_dim: Optional[int] = None
    ffn: int = 688
    rope_theta: float = 10000.0
    rms_eps: float = 1e-6
    qk_norm: bool = False
    tie_embeddings: bool = False
    init_std: float = 0.02
    name: str = "custom"

    def __post_init__(self):
        if self.head_dim is None:
            self.head_dim = self.hidden // self.n_heads

    @property
    def q_dim(self) -> int:
        return self.n_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.n_kv_heads * self.head_dim

    def num_params(self) -> int:
        per_layer = sum(n for _, (n, _s) in layer_param_specs(self).items())
        emb = self.vocab_size * self.hidden
        return self.n_layers * per_layer + emb * (1 if self.tie_embeddings else 2) + self.hidden


PRESETS: Dict[str, ModelConfig] = {
    # BASELINE config 1: CPU fp32 2-layer Llama-style decoder
    "tiny-llama": ModelConfig(1024, 256, 2, 4, 2, None, 688, 10000.0, 1e-6, False, False, 0.02, "tiny-llama"),
    "qwen3-4b": ModelConfig(151936, 2560, 36, 32, 8, 128, 9728, 1e6, 1e-6, True, True, 0.02, "qwen3-4b"),
    "llama3-8b": ModelConfig(128256, 4096, 32, 32, 8, 128, 14336, 5e5, 1e-5, False, False, 0.02, "llama3-8b"),
    "qwen3-0.6b": ModelConfig(151936, 1024, 28, 16, 8, 128, 3072, 1e6, 1e-6, True, True, 0.02, "qwen3-0.6b"),
    "qwen3-1.7b": ModelConfig(151936, 2048, 28, 16, 8, 128, 6144, 1e6, 1e-6, True, True, 0.02, "qwen3-1.7b"),
}


def get_config(name: str, **overrides) -> ModelConfig:
    base = PRESETS[name]
    d = dict(base.__dict__)
    d.update(overrides)
    return ModelConfig(**d)


def layer_param_specs(cfg: ModelConfig) -> Dict[str, Tuple[int, Tuple[int, ...]]]:
    """Ordered ``name -> (numel, shape)`` of one layer's parameters inside its flat buffer."""
    H, F_, q, kv, hd = cfg.hidden, cfg.ffn, cfg.q_dim, cfg.kv_dim, cfg.head_dim
    specs = [
        ("self_attn.q_proj.weight", (q, H)),
        ("self_attn.k_proj.weight", (kv, H)),
        ("self_attn.v_proj.weight", (kv, H)),
        ("self_attn.o_proj.weight", (H, q)),
        ("mlp.gate_proj.weight", (F_, H)),
        ("mlp.up_proj.weight", (F_, H)),
        ("mlp.down_proj.weight", (H, F_)),
        ("input_layernorm.weight", (H,)),
        ("post_attention_layernorm.weight", (H,)),
    ]
    if cfg.qk_norm:
        specs += [("self_attn.q_norm.weight", (hd,)), ("self_attn.k_norm.weight", (hd,))]
    return {n: (int(math.prod(s)), s) for n, s in specs}


def layer_views(cfg: ModelConfig, flat: torch.Tensor) -> Dict[str, torch.Tensor]:
    """Named views (plus the fused ``wqkv`` / ``wgu``) into one layer's flat buffer."""
    out, off = {}, 0
    for name, (n, shape) in layer_param_specs(cfg).items():
        out[name] = flat[off:off + n].view(shape)
        off += n
    H = cfg.hidden
    qkv_rows = cfg.q_dim + 2 * cfg.kv_dim
    out["wqkv"] = flat[0:qkv_rows * H].view(qkv_rows, H)
    o_end = qkv_rows * H + H * cfg.q_dim
    out["wgu"] = flat[o_end:o_end + 2 * cfg.ffn * H].view(2 * cfg.ffn, H)
    return out


def layer_numel(cfg: ModelConfig) -> int:
    return sum(n for n, _ in layer_param_specs(cfg).values())


# --------------------------------------------------------------------------
# manual layer forward / backward (kernels)
# --------------------------------------------------------------------------
def layer_forward(cfg: ModelConfig, w: Dict[str, torch.Tensor], x: torch.Tensor, cos, sin,
                  save: bool = True, qkv_fn=None):
    """x: [B, S, H].  Returns (y, saved).  ``qkv_fn(h1) -> [T, q + 2kv]`` replaces the fused QKV
    projection (the sharded runtime passes its all-gather-fused GEMM here)."""
    B, S, H = x.shape
    T = B * S
    hd, nq, nkv = cfg.head_dim, cfg.n_heads, cfg.n_kv_heads
    x2d = x.reshape(T, H)
    h1, rstd1 = M.rmsnorm_fwd(x2d, w["input_layernorm.weight"], cfg.rms_eps)
    qkv = qkv_fn(h1) if qkv_fn is not None else G.mm_nt(h1, w["wqkv"])   # [T, q + 2kv]
    q = qkv[:, :cfg.q_dim].reshape(B, S, nq, hd)
    k = qkv[:, cfg.q_dim:cfg.q_dim + cfg.kv_dim].reshape(B, S, nkv, hd)
    v = qkv[:, cfg.q_dim + cfg.kv_dim:].reshape(B, S, nkv, hd)
    qn_ctx = None
    if cfg.qk_norm:
        qc, kc = q.contiguous(), k.contiguous()
        qn, q_rstd = M.rmsnorm_fwd(qc, w["self_attn.q_norm.weight"], cfg.rms_eps)
        kn, k_rstd = M.rmsnorm_fwd(kc, w["self_attn.k_norm.weight"], cfg.rms_eps)
        qn_ctx = (qc, q_rstd, kc, k_rstd)
        q, k = qn, kn
        M.rope_(q, cos, sin)
        M.rope_(k, cos, sin)
    else:
        # rotate straight out of the fused projection buffer (no separate unpacking copy)
        qr = torch.empty(B, S, nq, hd, dtype=qkv.dtype, device=qkv.device)
        kr = torch.empty(B, S, nkv, hd, dtype=qkv.dtype, device=qkv.device)
        M.rope_into(qr.view(T, cfg.q_dim), qkv[:, :cfg.q_dim], cos, sin, S, nq, hd)
        M.rope_into(kr.view(T, cfg.kv_dim), qkv[:, cfg.q_dim:cfg.q_dim + cfg.kv_dim], cos, sin, S, nkv, hd)
        q, k = qr, kr
    a, actx = M.attention_fwd(q, k, v)
    a2d = a.reshape(T, cfg.q_dim)
    x2 = G.mm_nt_add(a2d, w["self_attn.o_proj.weight"], x2d)       # residual add in the epilogue
    h2, rstd2 = M.rmsnorm_fwd(x2, w["post_attention_layernorm.weight"], cfg.rms_eps)
    gu, act = G.mlp_gate_up(h2, w["wgu"])                           # [T, 2F], silu(gate) * up fused
    y = G.mm_nt_add(act, w["mlp.down_proj.weight"], x2)
    saved = None
    if save:
        saved = dict(x=x2d, rstd1=rstd1, h1=h1, qn=qn_ctx, actx=actx, a=a2d, x2=x2, rstd2=rstd2,
                     h2=h2, gu=gu, act=act, shape=(B, S, H))
    return y.reshape(B, S, H), saved


def layer_backward(cfg: ModelConfig, w: Dict[str, torch.Tensor], gw: Dict[str, torch.Tensor],
                   saved, dy: torch.Tensor, cos, sin, accumulate: bool = False) -> torch.Tensor:
    """Writes (or accumulates) the layer's weight gradients into ``gw`` views; returns dx."""
    B, S, H = saved["shape"]
    T = B * S
    hd, nq, nkv = cfg.head_dim, cfg.n_heads, cfg.n_kv_heads
    dy2 = dy.reshape(T, H)

    def put(name, val):
        if accumulate:
            gw[name].add_(val.to(gw[name].dtype).view(gw[name].shape))
        else:
            gw[name].copy_(val.view(gw[name].shape))
            if G.grad_sumsq() is not None:
                G.add_sumsq(gw[name], G.grad_sumsq())

    def wgrad(name, a, b):
        # a^T @ b straight into the gradient view (no temporary) unless accumulating; while a
        # gradient-norm accumulator is set, the product's epilogue also sums the squares it stores
        if accumulate:
            gw[name].add_(G.mm_tn(a, b))
        else:
            G.mm_tn_wgrad(a, b, gw[name])

    # MLP
    wgrad("mlp.down_proj.weight", dy2, saved["act"])
    dgu = G.mlp_down_dgrad(dy2, w["mlp.down_proj.weight"], saved["gu"])   # SwiGLU derivative fused
    wgrad("wgu", dgu, saved["h2"])
    dh2 = G.mm_nn(dgu, w["wgu"])
    # the residual branch's gradient (dy2) is added inside the norm's backward kernel
    dx2, dw = M.rmsnorm_bwd(dh2, saved["x2"], w["post_attention_layernorm.weight"], saved["rstd2"], res=dy2)
    put("post_attention_layernorm.weight", dw)
    # attention
    wgrad("self_attn.o_proj.weight", dx2, saved["a"])
    da = G.mm_nn(dx2, w["self_attn.o_proj.weight"]).reshape(B, S, nq, hd)
    dq, dk, dv = M.attention_bwd(saved["actx"], da)
    if cfg.qk_norm:
        dq, dk = dq.contiguous(), dk.contiguous()
        M.rope_(dq, cos, sin, inverse=True)
        M.rope_(dk, cos, sin, inverse=True)
        qc, q_rstd, kc, k_rstd = saved["qn"]
        dq, dwq = M.rmsnorm_bwd(dq, qc, w["self_attn.q_norm.weight"], q_rstd)
        dk, dwk = M.rmsnorm_bwd(dk, kc, w["self_attn.k_norm.weight"], k_rstd)
        put("self_attn.q_norm.weight", dwq)
        put("self_attn.k_norm.weight", dwk)
        dqkv = torch.cat((dq.reshape(T, -1), dk.reshape(T, -1), dv.reshape(T, -1)), dim=1)
    else:
        # inverse rotation written straight into the fused gradient buffer
        qd, kd = cfg.q_dim, cfg.kv_dim
        dqkv = torch.empty(T, qd + 2 * kd, dtype=dq.dtype, device=dq.device)
        M.rope_into(dqkv[:, :qd], dq.reshape(T, qd), cos, sin, S, nq, hd, inverse=True)
        M.rope_into(dqkv[:, qd:qd + kd], dk.reshape(T, kd), cos, sin, S, nkv, hd, inverse=True)
        dqkv[:, qd + kd:].copy_(dv.reshape(T, kd))
    wgrad("wqkv", dqkv, saved["h1"])
    dh1 = G.mm_nn(dqkv, w["wqkv"])
    dx, dw = M.rmsnorm_bwd(dh1, saved["x"], w["input_layernorm.weight"], saved["rstd1"], res=dx2)
    put("input_layernorm.weight", dw)
    return dx.reshape(B, S, H)


class _LayerFn(torch.autograd.Function):
    """One decoder layer as a single autograd node (manual backward).

    The layer's Parameters are passed as inputs so that autograd routes their
    gradients; they all alias ``flat`` (the layer's packed weight buffer), which
    is what the kernels read.  The gradients returned are row-slice views of one
    freshly written flat gradient buffer.
    """

    @staticmethod
    def forward(ctx, x, flat, cfg, cos, sin, *params):
        w = layer_views(cfg, flat)
        y, saved = layer_forward(cfg, w, x, cos, sin, save=True)
        ctx.cfg, ctx.saved, ctx.cos, ctx.sin = cfg, saved, cos, sin
        ctx.flat = flat
        return y

    @staticmethod
    def backward(ctx, dy):
        cfg = ctx.cfg
        flat = ctx.flat
        gflat = torch.empty_like(flat)
        w = layer_views(cfg, flat)
        gw = layer_views(cfg, gflat)
        dx = layer_backward(cfg, w, gw, ctx.saved, dy.contiguous(), ctx.cos, ctx.sin)
        ctx.saved = None
        grads = tuple(gw[name] for name in layer_param_specs(cfg))
        return (dx, None, None, None, None) + grads


# --------------------------------------------------------------------------
# plain torch layer (autograd) — CPU path and oracle
# --------------------------------------------------------------------------
def layer_forward_torch(cfg: ModelConfig, w: Dict[str, torch.Tensor], x: torch.Tensor, cos, sin):
    B, S, H = x.shape
    hd, nq, nkv = cfg.head_dim, cfg.n_heads, cfg.n_kv_heads

    def norm(t, weight):
        tf = t.float()
        return (tf * torch.rsqrt(tf.square().mean(-1, keepdim=True) + cfg.rms_eps) * weight.float()).to(t.dtype)

    def rope(t):
        h = hd // 2
        c, s = cos[None, :S, None, :].to(t.dtype), sin[None, :S, None, :].to(t.dtype)
        a, b = t[..., :h], t[..., h:]
        return torch.cat((a * c - b * s, b * c + a * s), dim=-1)

    h1 = norm(x, w["input_layernorm.weight"])
    q = F.linear(h1, w["self_attn.q_proj.weight"]).view(B, S, nq, hd)
    k = F.linear(h1, w["self_attn.k_proj.weight"]).view(B, S, nkv, hd)
    v = F.linear(h1, w["self_attn.v_proj.weight"]).view(B, S, nkv, hd)
    if cfg.qk_norm:
        q = norm(q, w["self_attn.q_norm.weight"])
        k = norm(k, w["self_attn.k_norm.weight"])
    q, k = rope(q), rope(k)
    rep = nq // nkv
    kk = k.repeat_interleave(rep, dim=2) if rep > 1 else k
    vv = v.repeat_interleave(rep, dim=2) if rep > 1 else v
    a = F.scaled_dot_product_attention(q.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2),
                                       is_causal=True).transpose(1, 2).reshape(B, S, nq * hd)
    x2 = x + F.linear(a, w["self_attn.o_proj.weight"])
    h2 = norm(x2, w["post_attention_layernorm.weight"])
    act = F.silu(F.linear(h2, w["mlp.gate_proj.weight"])) * F.linear(h2, w["mlp.up_proj.weight"])
    return x2 + F.linear(act, w["mlp.down_proj.weight"])


class DecoderLM(nn.Module):
    """Decoder-only LM with HF-style parameter names.

    ``forward(tokens, targets)`` returns the mean next-token cross-entropy when
    ``targets`` is given, else the logits.  ``impl="auto"`` uses the kernel path
    for CUDA half-precision weights and the plain torch path otherwise.

    Every matrix is its own ``nn.Parameter`` (``model.layers.0.self_attn.q_proj.weight``
    ...), and all Parameters of a layer are row-slice views of one packed buffer
    so that the fused QKV / gate-up GEMMs read them without a copy.
    """

    def __init__(self, cfg: ModelConfig, device=None, dtype=torch.float32, impl: str = "auto",
                 seed: Optional[int] = None):
        super().__init__()
        self.cfg = cfg
        self.impl = impl
        gen = None
        if seed is not None:
            gen = torch.Generator(device="cpu").manual_seed(seed)
        H, V = cfg.hidden, cfg.vocab_size

        def init(shape):
            t = torch.empty(shape, dtype=torch.float32)
            t.normal_(0.0, cfg.init_std, generator=gen)
            return t

        self.model = nn.Module()
        self.model.embed_tokens = nn.Embedding(V, H, device=device, dtype=dtype)
        with torch.no_grad():
            self.model.embed_tokens.weight.copy_(init((V, H)))
        self._flats: List[torch.Tensor] = []
        self.model.layers = nn.ModuleList()
        n = layer_numel(cfg)
        for _ in range(cfg.n_layers):
            flat = torch.empty(n, device=device, dtype=dtype)
            views = layer_views(cfg, flat)
            with torch.no_grad():
                for name, (_, shape) in layer_param_specs(cfg).items():
                    if name.endswith("norm.weight") or "layernorm" in name:
                        views[name].fill_(1.0)
                    else:
                        views[name].copy_(init(shape))
            self._flats.append(flat)
            self.model.layers.append(self._make_layer(views))
        self.model.norm = nn.Module()
        self.model.norm.weight = nn.Parameter(torch.ones(H, device=device, dtype=dtype))
        if cfg.tie_embeddings:
            self.lm_head = None
        else:
            self.lm_head = nn.Module()
            self.lm_head.weight = nn.Parameter(init((V, H)).to(device=device, dtype=dtype))
        self._rope_cache = {}

    def _make_layer(self, views: Dict[str, torch.Tensor]) -> nn.Module:
        layer = nn.Module()
        for name in layer_param_specs(self.cfg):
            parts = name.split(".")
            mod = layer
            for part in parts[:-1]:
                if not hasattr(mod, part):
                    setattr(mod, part, nn.Module())
                mod = getattr(mod, part)
            setattr(mod, parts[-1], nn.Parameter(views[name]))
        return layer

    def _layer_param(self, layer: nn.Module, name: str) -> nn.Parameter:
        obj = layer
        for part in name.split("."):
            obj = getattr(obj, part)
        return obj

    def _apply(self, fn, *args, **kwargs):
        """Device / dtype moves re-pack every layer so that its Parameters alias one buffer again."""
        out = super()._apply(fn, *args, **kwargs)
        with torch.no_grad():
            for i, layer in enumerate(self.model.layers):
                first = self._layer_param(layer, next(iter(layer_param_specs(self.cfg))))
                flat = torch.empty(layer_numel(self.cfg), device=first.device, dtype=first.dtype)
                views = layer_views(self.cfg, flat)
                for name in layer_param_specs(self.cfg):
                    p = self._layer_param(layer, name)
                    views[name].copy_(p.data)
                    p.data = views[name]
                self._flats[i] = flat
        self._rope_cache = {}
        return out

    # -- rope tables ------------------------------------------------------
    def rope(self, seq_len: int, device):
        key = (seq_len, str(device))
        if key not in self._rope_cache:
            self._rope_cache[key] = M.rope_tables(seq_len, self.cfg.head_dim, self.cfg.rope_theta, device)
        return self._rope_cache[key]

    def head_weight(self) -> torch.Tensor:
        return self.model.embed_tokens.weight if self.lm_head is None else self.lm_head.weight

    def _kernel_path(self, x: torch.Tensor) -> bool:
        if self.impl == "torch":
            return False
        if self.impl == "kernel":
            return True
        return x.is_cuda and x.dtype in (torch.bfloat16, torch.float16)

    def forward(self, tokens: torch.Tensor, targets: Optional[torch.Tensor] = None):
        cfg = self.cfg
        B, S = tokens.shape
        x = self.model.embed_tokens(tokens)
        cos, sin = self.rope(S, x.device)
        kernel = self._kernel_path(x)
        names = list(layer_param_specs(cfg))
        for flat, layer in zip(self._flats, self.model.layers):
            params = [self._layer_param(layer, n) for n in names]
            if kernel:
                x = _LayerFn.apply(x, flat, cfg, cos, sin, *params)
            else:
                x = layer_forward_torch(cfg, dict(zip(names, params)), x, cos, sin)
        xf = x.float()
        hN = (xf * torch.rsqrt(xf.square().mean(-1, keepdim=True) + cfg.rms_eps)
              * self.model.norm.weight.float()).to(x.dtype)
        logits = F.linear(hN, self.head_weight())
        if targets is None:
            return logits
        return F.cross_entropy(logits.float().view(B * S, -1), targets.reshape(-1))
