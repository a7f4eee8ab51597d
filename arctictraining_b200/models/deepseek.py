# SPDX-License-Identifier: Apache-2.0
"""DeepSeek-V2 family on the native stack: multi-head latent attention (MLA) and routed + shared experts.

MLA (as in the Hugging Face implementation, transformers/models/deepseek_v2/modeling_deepseek_v2.py, and the remote
code the reference vendors in projects/swiftkv/models/deepseek_v2/modeling_deepseek.py:620-800): queries come from a
(optionally low-rank) projection and have a ``qk_nope_head_dim`` part without position information and a
``qk_rope_head_dim`` rotary part; keys and values are up-projected from one ``kv_lora_rank`` latent per token, and all
heads share one rotary key taken straight from the down-projection.  The softmax scale is ``(nope + rope)^-0.5``,
times ``mscale^2`` under YaRN.

Native layout: parameter names equal the Hugging Face ones, but the rotary rows of ``q(_b)_proj`` and
``kv_a_proj_with_mqa`` are stored de-interleaved (even pair members first, then odd), so the rotate-half RoPE kernel
of this library applies; the permutation is applied when loading and undone when exporting, and cancels in
``q . k``.  Values are zero-padded to the query/key width for the attention call (one head width per call), so every
attention back end and the Ulysses exchange work unchanged.  MoE layers are ``ArcticMoE`` blocks (softmax -> top-k,
greedy or group-limited, unnormalised scores times ``routed_scaling_factor``, ungated shared experts), so they take
part in expert parallelism like the Qwen3-MoE ones.
"""

from __future__ import annotations

import re
from typing import Any
from typing import Dict
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..ops import reference as ref
from . import hf_io
from .arch import PRESETS
from .arch import ArchConfig
from .causal_lm import CausalLM
from .causal_lm import DecoderModel
from .modules import MLP
from .modules import DecoderLayer
from .modules import ForwardContext
from .modules import Linear
from .modules import RMSNorm
from .modules import _project_with_residual

LATENT_NORM_EPS = 1e-6


def mla_softmax_scale(cfg: ArchConfig) -> float:
    qk = cfg["qk_nope_head_dim"] + cfg["qk_rope_head_dim"]
    scale = qk ** -0.5
    rs = cfg.get("rope_scaling") or {}
    if rs.get("mscale_all_dim"):
        m = ref.yarn_mscale(float(rs.get("factor", 1.0)), float(rs["mscale_all_dim"]))
        scale *= m * m
    return scale


class MLAQuery(nn.Module):
    """The query branch: ``q_proj`` or ``q_a_proj -> q_a_layernorm -> q_b_proj``; output ``[B, S, heads, nope + rope]``
    with the rotary part rotated."""

    def __init__(self, cfg: ArchConfig, dtype=None, device=None) -> None:
        super().__init__()
        hidden, self.heads = cfg["hidden_size"], cfg["num_attention_heads"]
        self.nope, self.rope = cfg["qk_nope_head_dim"], cfg["qk_rope_head_dim"]
        rank = cfg.get("q_lora_rank")
        bias = bool(cfg.get("attention_bias", False))
        if rank:
            self.q_a_proj = Linear(hidden, rank, bias=bias, dtype=dtype, device=device)
            self.q_a_layernorm = RMSNorm(rank, LATENT_NORM_EPS, dtype=dtype, device=device)
            self.q_b_proj = Linear(rank, self.heads * (self.nope + self.rope), dtype=dtype, device=device)
        else:
            self.q_proj = Linear(hidden, self.heads * (self.nope + self.rope), dtype=dtype, device=device)

    def forward(self, x: torch.Tensor, ctx: ForwardContext) -> torch.Tensor:
        B, S, _ = x.shape
        q = self.q_b_proj(self.q_a_layernorm(self.q_a_proj(x))) if hasattr(self, "q_a_proj") else self.q_proj(x)
        q = q.view(B, S, self.heads, self.nope + self.rope)
        q_pe = ops.rope(q[..., self.nope :].contiguous(), ctx.cos, ctx.sin)
        return torch.cat([q[..., : self.nope], q_pe], dim=-1)


class MLAKeyValue(nn.Module):
    """The key/value branch: ``kv_a_proj_with_mqa -> (latent, shared rotary key)``, ``kv_a_layernorm``, ``kv_b_proj``.
    Returns keys ``[B, S, heads, nope + rope]`` and values ``[B, S, heads, v_head_dim]``."""

    def __init__(self, cfg: ArchConfig, dtype=None, device=None) -> None:
        super().__init__()
        hidden, self.heads = cfg["hidden_size"], cfg["num_attention_heads"]
        self.nope, self.rope, self.vd = cfg["qk_nope_head_dim"], cfg["qk_rope_head_dim"], cfg["v_head_dim"]
        self.rank = cfg["kv_lora_rank"]
        bias = bool(cfg.get("attention_bias", False))
        self.kv_a_proj_with_mqa = Linear(hidden, self.rank + self.rope, bias=bias, dtype=dtype, device=device)
        self.kv_a_layernorm = RMSNorm(self.rank, LATENT_NORM_EPS, dtype=dtype, device=device)
        self.kv_b_proj = Linear(self.rank, self.heads * (self.nope + self.vd), dtype=dtype, device=device)

    def forward(self, x: torch.Tensor, ctx: ForwardContext):
        B, S, _ = x.shape
        a = self.kv_a_proj_with_mqa(x)
        latent, k_pe = a[..., : self.rank], a[..., self.rank :]
        kv = self.kv_b_proj(self.kv_a_layernorm(latent.contiguous())).view(B, S, self.heads, self.nope + self.vd)
        k_pe = ops.rope(k_pe.reshape(B, S, 1, self.rope).contiguous(), ctx.cos, ctx.sin)
        k = torch.cat([kv[..., : self.nope], k_pe.expand(B, S, self.heads, self.rope)], dim=-1)
        return k, kv[..., self.nope :]


class MLAttention(nn.Module):
    def __init__(self, cfg: ArchConfig, layer_idx: int, dtype=None, device=None) -> None:
        super().__init__()
        self.layer_idx = layer_idx
        self.heads, self.vd = cfg["num_attention_heads"], cfg["v_head_dim"]
        self.qk = cfg["qk_nope_head_dim"] + cfg["qk_rope_head_dim"]
        self.scale = mla_softmax_scale(cfg)
        self.q = MLAQuery(cfg, dtype=dtype, device=device)
        self.kv = MLAKeyValue(cfg, dtype=dtype, device=device)
        self.o_proj = Linear(self.heads * self.vd, cfg["hidden_size"], bias=bool(cfg.get("attention_bias", False)),
                             dtype=dtype, device=device)

    def attend(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, ctx: ForwardContext) -> torch.Tensor:
        """Causal attention with value width ``v_head_dim <= qk width``: values are zero-padded to the query/key width
        and the padding columns of the output dropped."""
        B, S = q.shape[:2]
        if self.vd < self.qk:
            v = F.pad(v, (0, self.qk - self.vd))
        if ctx.kv_cache is not None:
            past = ctx.kv_cache[self.layer_idx]
            if past is not None:
                k, v = torch.cat([past[0], k], dim=1), torch.cat([past[1], v], dim=1)
            ctx.kv_cache[self.layer_idx] = (k, v)
            Sk = k.shape[1]
            mask = None
            if S > 1:
                mask = torch.arange(Sk, device=q.device).view(1, Sk) <= torch.arange(Sk - S, Sk, device=q.device).view(S, 1)
            o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attn_mask=mask,
                                               scale=self.scale).transpose(1, 2)
        elif ctx.sp is not None:
            o = ctx.sp.attention(q * (self.scale * self.qk ** 0.5), k, v, ctx)  # the exchange path uses the default scale
        else:
            o = ops.attention(q, k, v, ctx.cu_seqlens, ctx.max_seqlen, True, ctx.attn_impl, scale=self.scale)
        return o[..., : self.vd].reshape(B, S, self.heads * self.vd)

    def forward(self, x: torch.Tensor, ctx: ForwardContext, residual: Optional[torch.Tensor] = None,
                shared_kv=None, query: Optional[MLAQuery] = None) -> torch.Tensor:
        q = (query or self.q)(x, ctx)
        k, v = shared_kv if shared_kv is not None else self.kv(x, ctx)
        return _project_with_residual(self.o_proj, self.attend(q, k, v, ctx), residual)


class DeepseekDecoderLayer(DecoderLayer):
    attention_cls = MLAttention

    def __init__(self, cfg: ArchConfig, layer_idx: int, dtype=None, device=None) -> None:
        nn.Module.__init__(self)
        hidden = cfg["hidden_size"]
        self.layer_idx = layer_idx
        self.input_layernorm = RMSNorm(hidden, cfg["rms_norm_eps"], dtype=dtype, device=device)
        self.self_attn = self.attention_cls(cfg, layer_idx, dtype=dtype, device=device)
        self.post_attention_layernorm = RMSNorm(hidden, cfg["rms_norm_eps"], dtype=dtype, device=device)
        sparse = (cfg.get("n_routed_experts") and layer_idx >= int(cfg.get("first_k_dense_replace") or 0)
                  and layer_idx % int(cfg.get("moe_layer_freq") or 1) == 0)
        if sparse:
            from ..moe.layer import build_moe_block

            self.mlp = build_moe_block(cfg, dtype=dtype, device=device)
        else:
            self.mlp = MLP(hidden, cfg["intermediate_size"], dtype=dtype, device=device)

    def forward(self, x: torch.Tensor, ctx: ForwardContext, **attn_kw: Any) -> torch.Tensor:
        x = self.self_attn(self.input_layernorm(x), ctx, residual=x, **attn_kw)
        h = self.post_attention_layernorm(x)
        if type(self.mlp) is MLP:
            if ctx.tiled_mlp:
                from ..ops.tiled import tiled_mlp

                return x + tiled_mlp(self.mlp, h)
            return self.mlp(h, residual=x)
        return x + self.mlp(h)


class DeepseekDecoderModel(DecoderModel):
    layer_cls = DeepseekDecoderLayer

    def build_layer(self, cfg: ArchConfig, idx: int, dtype, device) -> nn.Module:
        return self.layer_cls(cfg, idx, dtype=dtype, device=device)

    def make_context(self, position_ids: torch.Tensor, attn_impl: str, **kw: Any) -> ForwardContext:
        cfg = self.cfg

        def rope_fn(pos: torch.Tensor):  # only the rotary part of a head is rotated
            return ref.rope_cos_sin(pos, int(cfg["qk_rope_head_dim"]), float(cfg.get("rope_theta") or 10000.0),
                                    cfg.get("rope_scaling"))

        cos, sin = rope_fn(position_ids)
        return ForwardContext(cos=cos, sin=sin, attn_impl=attn_impl, rope_fn=rope_fn, **kw)


class DeepseekV2ForCausalLM(CausalLM):
    decoder_cls = DeepseekDecoderModel


# ------------------------------------------------------------------------------------------------ HF names / layout
_ATTN_MOVED = re.compile(r"^(.*self_attn\.)(q_proj|q_a_proj|q_a_layernorm|q_b_proj)(_swiftkv)?\.(weight|bias)$")
_KV_MOVED = re.compile(r"^(.*self_attn\.)(kv_a_proj_with_mqa|kv_a_layernorm|kv_b_proj)\.(weight|bias)$")


def _is_mla(cfg) -> bool:
    return bool(cfg.get("kv_lora_rank")) and bool(cfg.get("qk_rope_head_dim"))


def _pair_order(n: int, inverse: bool = False) -> torch.Tensor:
    """Row order that turns interleaved rotary pairs ``(0,1),(2,3)...`` into halves ``(0..n/2-1 | n/2..n-1)``."""
    fwd = torch.cat([torch.arange(0, n, 2), torch.arange(1, n, 2)])
    return torch.argsort(fwd) if inverse else fwd


def permute_rotary_rows(t: torch.Tensor, cfg, kind: str, inverse: bool = False) -> torch.Tensor:
    """Re-order the rotary output rows of a query (``kind='q'``: per head, after the ``nope`` rows) or of the joint
    key/value down-projection (``kind='kv_a'``: the last ``rope`` rows)."""
    nope, rope = int(cfg["qk_nope_head_dim"]), int(cfg["qk_rope_head_dim"])
    order = _pair_order(rope, inverse).to(t.device)
    if kind == "q":
        heads = int(cfg["num_attention_heads"])
        v = t.reshape(heads, nope + rope, *t.shape[1:]).clone()
        v[:, nope:] = v[:, nope:][:, order]
        return v.reshape(t.shape)
    rank = int(cfg["kv_lora_rank"])
    out = t.clone()
    out[rank:] = t[rank:][order]
    return out


def _native_to_hf(name: str, tensor: torch.Tensor, cfg):
    if not _is_mla(cfg):
        return None
    m = re.match(r"^(.*self_attn\.)(q|kv)\.(.+)$", name)
    if not m:
        return None
    pre, _branch, rest = m.groups()
    if rest.startswith(("q_proj.", "q_b_proj.")):
        tensor = permute_rotary_rows(tensor, cfg, "q", inverse=True)
    elif rest.startswith("kv_a_proj_with_mqa."):
        tensor = permute_rotary_rows(tensor, cfg, "kv_a", inverse=True)
    return [(pre + rest, tensor)]


def _hf_to_native(hf: Dict[str, torch.Tensor], out: Dict[str, torch.Tensor], cfg) -> None:
    if not _is_mla(cfg):
        return
    for name in list(hf):
        m = _ATTN_MOVED.match(name)
        if m and not m.group(3):
            pre, mod, _sk, kind = m.groups()
            t = hf.pop(name)
            if mod in ("q_proj", "q_b_proj"):
                t = permute_rotary_rows(t, cfg, "q")
            out[f"{pre}q.{mod}.{kind}"] = t
            continue
        m = _KV_MOVED.match(name)
        if m:
            pre, mod, kind = m.groups()
            t = hf.pop(name)
            if mod == "kv_a_proj_with_mqa":
                t = permute_rotary_rows(t, cfg, "kv_a")
            out[f"{pre}kv.{mod}.{kind}"] = t


if _native_to_hf not in hf_io._EXTRA_NATIVE_TO_HF:
    hf_io._EXTRA_NATIVE_TO_HF.insert(0, _native_to_hf)
    hf_io._EXTRA_HF_TO_NATIVE.insert(0, _hf_to_native)


def _deepseek(hidden, layers, heads, inter, vocab, *, q_rank, kv_rank, nope, rope, vdim, experts, topk, moe_inter, shared,
              first_dense, **extra) -> Dict[str, Any]:
    cfg = dict(
        architectures=["DeepseekV2ForCausalLM"], model_type="deepseek_v2", hidden_size=hidden, num_hidden_layers=layers,
        num_attention_heads=heads, num_key_value_heads=heads, intermediate_size=inter, vocab_size=vocab,
        q_lora_rank=q_rank, kv_lora_rank=kv_rank, qk_nope_head_dim=nope, qk_rope_head_dim=rope, v_head_dim=vdim,
        head_dim=rope, n_routed_experts=experts, num_experts_per_tok=topk, moe_intermediate_size=moe_inter,
        n_shared_experts=shared, first_k_dense_replace=first_dense, moe_layer_freq=1, norm_topk_prob=False,
        routed_scaling_factor=1.0, topk_method="greedy", n_group=1, topk_group=1, aux_loss_alpha=0.001,
        rope_theta=10000.0, max_position_embeddings=163840, rms_norm_eps=1e-6, hidden_act="silu",
        tie_word_embeddings=False, attention_bias=False, mlp_bias=False, bos_token_id=100000, eos_token_id=100001,
        torch_dtype="bfloat16",
    )
    cfg.update(extra)
    return cfg


_YARN_V2 = dict(type="yarn", factor=40, original_max_position_embeddings=4096, beta_fast=32, beta_slow=1, mscale=0.707,
                mscale_all_dim=0.707)
PRESETS.setdefault("deepseek-v2-lite", _deepseek(
    2048, 27, 16, 10944, 102400, q_rank=None, kv_rank=512, nope=128, rope=64, vdim=128, experts=64, topk=6, moe_inter=1408,
    shared=2, first_dense=1, rope_scaling=dict(_YARN_V2)))
PRESETS.setdefault("deepseek-v2", _deepseek(
    5120, 60, 128, 12288, 102400, q_rank=1536, kv_rank=512, nope=128, rope=64, vdim=128, experts=160, topk=6, moe_inter=1536,
    shared=2, first_dense=1, routed_scaling_factor=16.0, topk_method="group_limited_greedy", n_group=8, topk_group=3,
    rope_scaling=dict(_YARN_V2)))
PRESETS.setdefault("tiny-deepseek-v2", _deepseek(
    64, 3, 4, 128, 1024, q_rank=24, kv_rank=16, nope=16, rope=8, vdim=16, experts=8, topk=2, moe_inter=64, shared=1,
    first_dense=1, max_position_embeddings=2048, bos_token_id=1, eos_token_id=2))
