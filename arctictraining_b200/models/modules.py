# SPDX-License-Identifier: Apache-2.0
"""Decoder building blocks shared by the native model families (Llama, Qwen2, Qwen3, Qwen3-MoE).

Weights of projections that are consumed together are stored fused — ``qkv_proj`` (q, k, v rows stacked)
and ``gate_up_proj`` (gate/up rows block-interleaved, 64 and 64) — so each is one GEMM whose epilogue can
apply RoPE or SwiGLU.  Conversion to and from the Hugging Face parameter names happens at checkpoint
load/save time (:mod:`arctictraining_b200.models.hf_io`).
"""

from __future__ import annotations

from dataclasses import dataclass
from dataclasses import field
from typing import Any
from typing import Dict
from typing import Optional

import torch
import torch.nn as nn

from .. import ops
from .arch import ArchConfig


@dataclass
class ForwardContext:
    """Per-batch tensors shared by all layers."""

    cos: torch.Tensor  # [B, S, D/2] fp32
    sin: torch.Tensor
    cu_seqlens: Optional[torch.Tensor] = None  # packed-sample boundaries over the *full* sequence
    max_seqlen: Optional[int] = None
    attn_impl: str = "sdpa"
    sp: Optional[Any] = None  # UlyssesContext when sequence parallelism is on
    tiled_mlp: bool = False
    extras: Dict[str, Any] = field(default_factory=dict)
    # rotary tables for arbitrary positions (used for the whole sequence when rotation happens after the Ulysses exchange)
    rope_fn: Optional[Any] = None
    # generation: one (keys, values) pair per layer, [B, S_past, Hkv, D], grown by every call (None: training / scoring)
    kv_cache: Optional[list] = None


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float, dtype=None, device=None) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.rms_norm(x, self.weight, self.eps)


class Linear(nn.Module):
    """``y = x W^T (+ b)`` on this library's GEMM.  ``weight`` is ``[out, in]`` like ``nn.Linear``."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, dtype=None, device=None) -> None:
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device)) if bias else None

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        return ops.linear(x, self.weight, self.bias, residual)


def _project_with_residual(proj: nn.Module, x: torch.Tensor, residual: Optional[torch.Tensor]) -> torch.Tensor:
    """``residual + proj(x)``; a plain :class:`Linear` fuses the addition, any wrapper (adapters) adds afterwards."""
    if residual is None:
        return proj(x)
    if type(proj) is Linear:
        return proj(x, residual)
    return residual + proj(x)


class Attention(nn.Module):
    def __init__(self, cfg: ArchConfig, layer_idx: int, dtype=None, device=None) -> None:
        super().__init__()
        self.layer_idx = layer_idx
        self.hq = cfg["num_attention_heads"]
        self.hkv = cfg.get("num_key_value_heads") or self.hq
        self.d = cfg.head_dim_
        hidden = cfg["hidden_size"]
        bias = bool(cfg.get("attention_bias", False))
        self.qkv_proj = Linear(hidden, (self.hq + 2 * self.hkv) * self.d, bias=bias, dtype=dtype, device=device)
        self.o_proj = Linear(self.hq * self.d, hidden, bias=False, dtype=dtype, device=device)
        # sliding-window layers (Qwen2: layers from ``max_window_layers`` on when ``use_sliding_window`` is set; Mistral:
        # every layer when ``sliding_window`` is given)
        self.window: Optional[int] = None
        sw = cfg.get("sliding_window")
        if sw and cfg.get("use_sliding_window", cfg.get("model_type") == "mistral"):
            if layer_idx >= int(cfg.get("max_window_layers", 0) or 0):
                self.window = int(sw)
        self.qk_norm = bool(cfg.get("qk_norm", False))
        if self.qk_norm:
            self.q_norm = RMSNorm(self.d, cfg["rms_norm_eps"], dtype=dtype, device=device)
            self.k_norm = RMSNorm(self.d, cfg["rms_norm_eps"], dtype=dtype, device=device)

    def project_qkv(self, x: torch.Tensor, ctx: ForwardContext):
        B, S, _ = x.shape
        qkv = self.qkv_proj(x)
        if self.qk_norm:
            q, k, v = qkv.split([self.hq * self.d, self.hkv * self.d, self.hkv * self.d], dim=-1)
            q = self.q_norm(q.reshape(B, S, self.hq, self.d))
            k = self.k_norm(k.reshape(B, S, self.hkv, self.d))
            q = ops.rope(q, ctx.cos, ctx.sin)
            k = ops.rope(k, ctx.cos, ctx.sin)
            v = v.reshape(B, S, self.hkv, self.d)
        else:
            q, k, v = ops.rope_qkv(qkv, ctx.cos, ctx.sin, self.hq, self.hkv, self.d)
        return q, k, v

    def core(self, q, k, v, ctx: ForwardContext) -> torch.Tensor:
        if ctx.sp is not None:
            return ctx.sp.attention(q, k, v, ctx)
        return ops.attention(q, k, v, ctx.cu_seqlens, ctx.max_seqlen, True, ctx.attn_impl, window=self.window)

    def _forward_cached(self, x: torch.Tensor, ctx: ForwardContext, residual: Optional[torch.Tensor]) -> torch.Tensor:
        """Generation step: the new tokens' keys and values are appended to the layer's cache and the queries attend to
        everything cached so far (causally among the new tokens when a whole prompt is processed at once)."""
        import torch.nn.functional as F

        B, S, _ = x.shape
        q, k, v = self.project_qkv(x, ctx)
        past = ctx.kv_cache[self.layer_idx]
        if past is not None:
            k = torch.cat([past[0], k], dim=1)
            v = torch.cat([past[1], v], dim=1)
        ctx.kv_cache[self.layer_idx] = (k, v)
        Sk = k.shape[1]
        mask = None
        if S > 1:
            qpos = torch.arange(Sk - S, Sk, device=x.device).view(S, 1)
            mask = torch.arange(Sk, device=x.device).view(1, Sk) <= qpos
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attn_mask=mask,
                                           enable_gqa=(self.hq != self.hkv))
        return _project_with_residual(self.o_proj, o.transpose(1, 2).reshape(B, S, self.hq * self.d), residual)

    def forward(self, x: torch.Tensor, ctx: ForwardContext, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        B, S, _ = x.shape
        if ctx.kv_cache is not None:
            return self._forward_cached(x, ctx, residual)
        if (
            ctx.sp is not None and hasattr(ctx.sp, "fused_attention_block") and not self.qk_norm
            and type(self.qkv_proj) is Linear and self.qkv_proj.bias is None
            and type(self.o_proj) is Linear and self.o_proj.bias is None
        ):
            fused = ctx.sp.fused_attention_block(x, self.qkv_proj.weight, self.o_proj.weight, ctx, self.hq, self.hkv, self.d, residual)
            if fused is not None:
                return fused
        if ctx.sp is None and not self.qk_norm and self.window is None and ctx.attn_impl == "native":
            # rotary embedding + attention as one autograd node on the fused projection output
            o = ops.rope_attention(self.qkv_proj(x), ctx.cos, ctx.sin, self.hq, self.hkv, self.d, ctx.cu_seqlens, ctx.max_seqlen)
            if o is not None:
                return _project_with_residual(self.o_proj, o.reshape(B, S, self.hq * self.d), residual)
        q, k, v = self.project_qkv(x, ctx)
        if ctx.sp is not None and type(self.o_proj) is Linear and self.o_proj.bias is None and hasattr(ctx.sp, "attention_project"):
            fused = ctx.sp.attention_project(q, k, v, ctx, self.o_proj.weight, residual)
            if fused is not None:
                return fused
        o = self.core(q, k, v, ctx)
        return _project_with_residual(self.o_proj, o.reshape(B, S, self.hq * self.d), residual)


class MLP(nn.Module):
    """SwiGLU feed-forward block with a fused, block-interleaved gate/up weight."""

    def __init__(self, hidden: int, inter: int, dtype=None, device=None) -> None:
        super().__init__()
        self.gate_up_proj = Linear(hidden, 2 * inter, dtype=dtype, device=device)
        self.down_proj = Linear(inter, hidden, dtype=dtype, device=device)

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
        if type(self.down_proj) is Linear and type(self.gate_up_proj) is Linear:
            return ops.mlp_swiglu(x, self.gate_up_proj.weight, self.down_proj.weight, residual)
        return _project_with_residual(self.down_proj, ops.linear_swiglu(x, self.gate_up_proj.weight), residual)


class DecoderLayer(nn.Module):
    def __init__(self, cfg: ArchConfig, layer_idx: int, dtype=None, device=None) -> None:
        super().__init__()
        hidden = cfg["hidden_size"]
        self.layer_idx = layer_idx
        self.input_layernorm = RMSNorm(hidden, cfg["rms_norm_eps"], dtype=dtype, device=device)
        self.self_attn = Attention(cfg, layer_idx, dtype=dtype, device=device)
        self.post_attention_layernorm = RMSNorm(hidden, cfg["rms_norm_eps"], dtype=dtype, device=device)
        self.mlp = self._build_mlp(cfg, layer_idx, dtype, device)

    @staticmethod
    def _build_mlp(cfg: ArchConfig, layer_idx: int, dtype, device) -> nn.Module:
        n_exp = cfg.get("num_experts") or cfg.get("num_local_experts") or 0
        sparse_step = cfg.get("decoder_sparse_step", 1) or 1
        if n_exp and layer_idx not in (cfg.get("mlp_only_layers") or []) and (layer_idx + 1) % sparse_step == 0:
            from ..moe.layer import build_moe_block

            return build_moe_block(cfg, dtype=dtype, device=device)
        return MLP(cfg["hidden_size"], cfg["intermediate_size"], dtype=dtype, device=device)

    def forward(self, x: torch.Tensor, ctx: ForwardContext) -> torch.Tensor:
        if type(self.self_attn) is Attention:
            x = self.self_attn(self.input_layernorm(x), ctx, residual=x)
        else:
            x = x + self.self_attn(self.input_layernorm(x), ctx)
        h = self.post_attention_layernorm(x)
        if ctx.tiled_mlp and isinstance(self.mlp, MLP):
            from ..ops.tiled import tiled_mlp

            return x + tiled_mlp(self.mlp, h)
        if type(self.mlp) is MLP:
            return self.mlp(h, residual=x)
        return x + self.mlp(h)
