# SPDX-License-Identifier: Apache-2.0
"""SwiftKV self-distillation on the native decoder.

Behaviour parity: projects/swiftkv/train.py:46-264 and projects/swiftkv/models/llama/modeling_llama_swiftkv.py:
(Llama / Qwen2 / Mistral families; the DeepSeek-V2 variant with latent attention is further down)
layers ``>= num_key_value_layers`` get an extra query projection (``q_proj_swiftkv``), every
``key_value_group_size``-th of them extra key/value projections (``k_proj_swiftkv`` / ``v_proj_swiftkv``); at layer
``num_key_value_layers`` the hidden state is normalised by ``norm_swiftkv`` and the keys/values of *all* later
layers are projected from that single tensor.  The teacher is the same network with SwiftKV switched off (no
gradient); only the SwiftKV parameters train.  Initialisation: queries copied from the teacher, keys/values =
mean of the teacher projections in the group, norm copied from the first SwiftKV layer.  Loss: temperature-scaled
KL on the logits of assistant tokens (tiled, fused kernel) + ``hidden_loss_mult`` x MSE on one hidden layer.

Native design points: the shared K/V projections live in one module (`swiftkv_kv`) that is its own engine unit, so
ZeRO-3 can gather it independently of the checkpointed layers that consume its output; shared K/V enter those layers
as differentiable inputs of the checkpointed unit; and the student starts from the teacher's hidden state at layer
``num_key_value_layers`` because the layers before it are frozen and identical in both networks.
"""

from __future__ import annotations

from typing import Any
from typing import Dict
from typing import List
from typing import Optional
from typing import Union

import torch
import torch.nn as nn
import torch.nn.functional as F

from arctictraining_b200 import ops
from arctictraining_b200.checkpoint.hf import HFCheckpointEngine
from arctictraining_b200.checkpoint.sharded import DSCheckpointEngine
from arctictraining_b200.config.model import ModelConfig
from arctictraining_b200.config.trainer import TrainerConfig
from arctictraining_b200.models import hf_io
from arctictraining_b200.models.causal_lm import CausalLM
from arctictraining_b200.models.causal_lm import DecoderModel
from arctictraining_b200.models.deepseek import DeepseekDecoderLayer
from arctictraining_b200.models.deepseek import DeepseekDecoderModel
from arctictraining_b200.models.deepseek import MLAKeyValue
from arctictraining_b200.models.deepseek import MLAQuery
from arctictraining_b200.models.deepseek import MLAttention
from arctictraining_b200.models.deepseek import permute_rotary_rows
from arctictraining_b200.models.factory import HFModelFactory
from arctictraining_b200.models.modules import Attention
from arctictraining_b200.models.modules import DecoderLayer
from arctictraining_b200.models.modules import ForwardContext
from arctictraining_b200.models.modules import Linear
from arctictraining_b200.models.modules import RMSNorm
from arctictraining_b200.ops import _ext
from arctictraining_b200.ops.functional import _count
from arctictraining_b200.ops.functional import _gemm_ok
from arctictraining_b200.ops.functional import _use_kernels
from arctictraining_b200.ops.functional import gemm
from arctictraining_b200.trainer.sft import SFTTrainer
from arctictraining_b200.trainer.utils import to_device


# ------------------------------------------------------------------------------------------------ model
class SwiftKVAttention(Attention):
    def __init__(self, cfg, layer_idx: int, dtype=None, device=None) -> None:
        super().__init__(cfg, layer_idx, dtype=dtype, device=device)
        nkv = cfg.get("num_key_value_layers") or cfg["num_hidden_layers"]
        self.is_swiftkv_layer = layer_idx >= nkv
        if self.is_swiftkv_layer:
            self.q_proj_swiftkv = Linear(cfg["hidden_size"], self.hq * self.d, bias=bool(cfg.get("attention_bias")),
                                         dtype=dtype, device=device)

    def forward(self, x, ctx: ForwardContext, k_shared=None, v_shared=None):
        if k_shared is None:
            return super().forward(x, ctx)
        B, S, _ = x.shape
        q = ops.rope(self.q_proj_swiftkv(x).view(B, S, self.hq, self.d), ctx.cos, ctx.sin)
        o = self.core(q, k_shared, v_shared, ctx)
        return self.o_proj(o.reshape(B, S, self.hq * self.d))


class SwiftKVDecoderLayer(DecoderLayer):
    def __init__(self, cfg, layer_idx: int, dtype=None, device=None) -> None:
        super().__init__(cfg, layer_idx, dtype=dtype, device=device)
        self.self_attn = SwiftKVAttention(cfg, layer_idx, dtype=dtype, device=device)

    def forward(self, x, ctx: ForwardContext, k_shared=None, v_shared=None):
        x = x + self.self_attn(self.input_layernorm(x), ctx, k_shared, v_shared)
        return x + self.mlp(self.post_attention_layernorm(x))


class SwiftKVProjector(nn.Module):
    """``norm_swiftkv`` and the fused K/V projections of every KV group, applied to one hidden state."""

    def __init__(self, cfg, dtype=None, device=None) -> None:
        super().__init__()
        self.nkv = cfg.get("num_key_value_layers") or cfg["num_hidden_layers"]
        self.group = max(1, int(cfg.get("key_value_group_size", 1)))
        self.hkv = cfg.get("num_key_value_heads") or cfg["num_attention_heads"]
        self.d = cfg.head_dim_
        n_layers = cfg["num_hidden_layers"]
        self.owner_layers = list(range(self.nkv, n_layers, self.group))
        self.norm_swiftkv = RMSNorm(cfg["hidden_size"], cfg["rms_norm_eps"], dtype=dtype, device=device)
        self.kv_proj = nn.ModuleList(
            [Linear(cfg["hidden_size"], 2 * self.hkv * self.d, bias=bool(cfg.get("attention_bias")), dtype=dtype, device=device)
             for _ in self.owner_layers]
        )

    def forward(self, hidden: torch.Tensor, ctx: ForwardContext) -> Dict[int, Any]:
        B, S, _ = hidden.shape
        h = self.norm_swiftkv(hidden)
        out: Dict[int, Any] = {}
        for proj, first in zip(self.kv_proj, self.owner_layers):
            kv = proj(h)
            k, v = kv.split([self.hkv * self.d, self.hkv * self.d], dim=-1)
            k = ops.rope(k.reshape(B, S, self.hkv, self.d), ctx.cos, ctx.sin)
            v = v.reshape(B, S, self.hkv, self.d)
            for layer_idx in range(first, first + self.group):
                out[layer_idx] = (k, v)
        return out


class SwiftKVDecoderModel(DecoderModel):
    projector_cls = SwiftKVProjector

    def __init__(self, cfg, dtype=None, device=None) -> None:
        super().__init__(cfg, dtype=dtype, device=device)
        self.swiftkv_kv = self.projector_cls(cfg, dtype=dtype, device=device)
        self.swiftkv_enabled = False

    def build_layer(self, cfg, idx: int, dtype, device) -> nn.Module:
        return SwiftKVDecoderLayer(cfg, idx, dtype=dtype, device=device)

    def run_layers(self, h: torch.Tensor, ctx: ForwardContext, start: int = 0, collect: Optional[List] = None):
        nkv = self.swiftkv_kv.nkv
        shared: Dict[int, Any] = {}
        for idx in range(start, len(self.layers)):
            if collect is not None:
                collect.append(h)
            if self.swiftkv_enabled and idx == nkv:
                shared = self.swiftkv_kv(h, ctx)
            if idx in shared:
                k, v = shared[idx]
                h = self.layers[idx](h, ctx, k, v)
            else:
                h = self.layers[idx](h, ctx)
        h = self.norm(h)
        if collect is not None:
            collect.append(h)
        return h

    def forward(self, input_ids, position_ids=None, ctx=None, output_hidden_states: bool = False, **_: Any):
        B, S = input_ids.shape
        if position_ids is None:
            position_ids = torch.arange(S, device=input_ids.device).unsqueeze(0).expand(B, S)
        if ctx is None:
            ctx = self.make_context(position_ids, "sdpa")
        collect: Optional[List] = [] if output_hidden_states else None
        h = self.run_layers(self.embed_tokens(input_ids), ctx, 0, collect)
        return (h, collect) if output_hidden_states else h


# ------------------------------------------------------------------------------------------------ DeepSeek-V2 (MLA)
class MLASwiftKVAttention(MLAttention):
    """Parity: projects/swiftkv/models/deepseek_v2/modeling_deepseek_swiftkv.py:55-188 — SwiftKV layers get a second
    query branch (``q_proj_swiftkv`` or ``q_a_proj_swiftkv / q_a_layernorm_swiftkv / q_b_proj_swiftkv``)."""

    def __init__(self, cfg, layer_idx: int, dtype=None, device=None) -> None:
        super().__init__(cfg, layer_idx, dtype=dtype, device=device)
        nkv = cfg.get("num_key_value_layers") or cfg["num_hidden_layers"]
        self.is_swiftkv_layer = layer_idx >= nkv
        if self.is_swiftkv_layer:
            self.q_swiftkv = MLAQuery(cfg, dtype=dtype, device=device)

    def forward(self, x, ctx: ForwardContext, residual=None, k_shared=None, v_shared=None):
        if k_shared is None:
            return super().forward(x, ctx, residual)
        return super().forward(x, ctx, residual, shared_kv=(k_shared, v_shared), query=self.q_swiftkv)


class MLASwiftKVDecoderLayer(DeepseekDecoderLayer):
    attention_cls = MLASwiftKVAttention

    def forward(self, x, ctx: ForwardContext, k_shared=None, v_shared=None):
        return super().forward(x, ctx, k_shared=k_shared, v_shared=v_shared)


class MLASwiftKVProjector(nn.Module):
    """``norm_swiftkv`` and one latent key/value branch (``kv_a_proj_with_mqa_swiftkv``, ``kv_a_layernorm_swiftkv``,
    ``kv_b_proj_swiftkv``) per KV group, applied to the hidden state that enters layer ``num_key_value_layers``."""

    def __init__(self, cfg, dtype=None, device=None) -> None:
        super().__init__()
        self.nkv = cfg.get("num_key_value_layers") or cfg["num_hidden_layers"]
        self.group = max(1, int(cfg.get("key_value_group_size", 1)))
        self.owner_layers = list(range(self.nkv, cfg["num_hidden_layers"], self.group))
        self.norm_swiftkv = RMSNorm(cfg["hidden_size"], cfg["rms_norm_eps"], dtype=dtype, device=device)
        self.kv_proj = nn.ModuleList([MLAKeyValue(cfg, dtype=dtype, device=device) for _ in self.owner_layers])

    def forward(self, hidden: torch.Tensor, ctx: ForwardContext) -> Dict[int, Any]:
        h = self.norm_swiftkv(hidden)
        out: Dict[int, Any] = {}
        for branch, first in zip(self.kv_proj, self.owner_layers):
            kv = branch(h, ctx)
            for layer_idx in range(first, first + self.group):
                out[layer_idx] = kv
        return out


class MLASwiftKVDecoderModel(SwiftKVDecoderModel):
    projector_cls = MLASwiftKVProjector
    make_context = DeepseekDecoderModel.make_context

    def build_layer(self, cfg, idx: int, dtype, device) -> nn.Module:
        return MLASwiftKVDecoderLayer(cfg, idx, dtype=dtype, device=device)


class SwiftKVForCausalLM(CausalLM):
    decoder_cls = SwiftKVDecoderModel

    def swiftkv(self, flag: bool) -> None:
        self.model.swiftkv_enabled = bool(flag)

    def zero_units(self):
        units = super().zero_units()
        units.insert(len(units) - 1, ("swiftkv_kv", [self.model.swiftkv_kv], False))
        return units


class MLASwiftKVForCausalLM(SwiftKVForCausalLM):
    decoder_cls = MLASwiftKVDecoderModel


# -- HF names: model.layers.N.self_attn.{k,v}_proj_swiftkv.weight <-> model.swiftkv_kv.kv_proj.<g>.weight -------------
_MLA_Q = ("q_proj", "q_a_proj", "q_a_layernorm", "q_b_proj")
_MLA_KV = ("kv_a_proj_with_mqa", "kv_a_layernorm", "kv_b_proj")


def _mla_native_to_hf(name: str, tensor: torch.Tensor, cfg):
    """``self_attn.q_swiftkv.<m>`` -> ``self_attn.<m>_swiftkv``; ``swiftkv_kv.kv_proj.<g>.<m>`` ->
    ``layers.<first layer of group g>.self_attn.<m>_swiftkv``; rotary rows back to the interleaved order."""
    if ".self_attn.q_swiftkv." in name:
        pre, rest = name.split("q_swiftkv.")
        mod, kind = rest.rsplit(".", 1)
        if mod in ("q_proj", "q_b_proj"):
            tensor = permute_rotary_rows(tensor, cfg, "q", inverse=True)
        return [(f"{pre}{mod}_swiftkv.{kind}", tensor)]
    if ".swiftkv_kv.kv_proj." in name:
        g, mod, kind = name.split(".swiftkv_kv.kv_proj.")[1].split(".")
        nkv = cfg.get("num_key_value_layers") or cfg["num_hidden_layers"]
        layer = nkv + int(g) * max(1, int(cfg.get("key_value_group_size", 1)))
        if mod == "kv_a_proj_with_mqa":
            tensor = permute_rotary_rows(tensor, cfg, "kv_a", inverse=True)
        return [(f"model.layers.{layer}.self_attn.{mod}_swiftkv.{kind}", tensor)]
    if name == "model.swiftkv_kv.norm_swiftkv.weight":
        return [("model.norm_swiftkv.weight", tensor)]
    return None


def _mla_hf_to_native(hf: Dict[str, torch.Tensor], out: Dict[str, torch.Tensor], cfg) -> None:
    nkv = cfg.get("num_key_value_layers")
    group = max(1, int(cfg.get("key_value_group_size", 1)))
    for name in list(hf):
        if "_swiftkv." not in name or ".self_attn." not in name:
            continue
        pre, rest = name.split("self_attn.")
        mod, kind = rest.rsplit(".", 1)
        mod = mod[: -len("_swiftkv")]
        t = hf.pop(name)
        if mod in _MLA_Q:
            if mod in ("q_proj", "q_b_proj"):
                t = permute_rotary_rows(t, cfg, "q")
            out[f"{pre}self_attn.q_swiftkv.{mod}.{kind}"] = t
        elif mod in _MLA_KV:
            layer = int(name.split("model.layers.")[1].split(".")[0])
            if mod == "kv_a_proj_with_mqa":
                t = permute_rotary_rows(t, cfg, "kv_a")
            out[f"model.swiftkv_kv.kv_proj.{(layer - nkv) // group}.{mod}.{kind}"] = t
    if "model.norm_swiftkv.weight" in hf:
        out["model.swiftkv_kv.norm_swiftkv.weight"] = hf.pop("model.norm_swiftkv.weight")


def _native_to_hf(name: str, tensor: torch.Tensor, cfg):
    if cfg.get("kv_lora_rank"):
        return _mla_native_to_hf(name, tensor, cfg)
    if ".swiftkv_kv.kv_proj." in name:
        g = int(name.split(".swiftkv_kv.kv_proj.")[1].split(".")[0])
        kind = name.rsplit(".", 1)[1]
        nkv = cfg.get("num_key_value_layers") or cfg["num_hidden_layers"]
        layer = nkv + g * max(1, int(cfg.get("key_value_group_size", 1)))
        k, v = tensor.chunk(2, dim=0)
        pre = f"model.layers.{layer}.self_attn."
        return [(f"{pre}k_proj_swiftkv.{kind}", k), (f"{pre}v_proj_swiftkv.{kind}", v)]
    if name == "model.swiftkv_kv.norm_swiftkv.weight":
        return [("model.norm_swiftkv.weight", tensor)]
    return None


def _hf_to_native(hf: Dict[str, torch.Tensor], out: Dict[str, torch.Tensor], cfg) -> None:
    nkv = cfg.get("num_key_value_layers")
    if nkv is None:
        return
    if cfg.get("kv_lora_rank"):
        return _mla_hf_to_native(hf, out, cfg)
    group = max(1, int(cfg.get("key_value_group_size", 1)))
    for name in list(hf):
        if name.endswith("k_proj_swiftkv.weight") or name.endswith("k_proj_swiftkv.bias"):
            kind = name.rsplit(".", 1)[1]
            layer = int(name.split("model.layers.")[1].split(".")[0])
            v = hf.pop(name.replace("k_proj_swiftkv", "v_proj_swiftkv"))
            out[f"model.swiftkv_kv.kv_proj.{(layer - nkv) // group}.{kind}"] = torch.cat([hf.pop(name), v], dim=0)
    if "model.norm_swiftkv.weight" in hf:
        out["model.swiftkv_kv.norm_swiftkv.weight"] = hf.pop("model.norm_swiftkv.weight")


if _native_to_hf not in hf_io._EXTRA_NATIVE_TO_HF:
    # ahead of the family converters: the SwiftKV names are a superset of theirs
    hf_io._EXTRA_NATIVE_TO_HF.insert(0, _native_to_hf)
    hf_io._EXTRA_HF_TO_NATIVE.insert(0, _hf_to_native)


# ------------------------------------------------------------------------------------------------ configs / factory
class SwiftKVModelConfig(ModelConfig):
    num_key_value_layers: int
    """ Number of leading layers that keep their own KV; the input of layer ``num_key_value_layers`` feeds the KV
    of all later layers. """

    key_value_group_size: int = 1
    """ Consecutive SwiftKV layers that share one KV projection. """


class SwiftKVTrainerConfig(TrainerConfig):
    logits_loss_temp: float = 2.0
    """ Temperature of the KL distillation loss on the logits. """

    hidden_loss_mult: float = 1.0
    """ Weight of the MSE loss on hidden states. """

    hidden_loss_layer: int = -2
    """ Index into the list of hidden states used for the hidden loss. """


class SwiftKVModelFactory(HFModelFactory):
    name = "swiftkv"
    config: SwiftKVModelConfig
    model_cls = SwiftKVForCausalLM

    def post_create_config_callback(self, hf_config):
        if hf_config.get("model_type") not in ("llama", "qwen2", "qwen3", "mistral", "deepseek_v2"):
            raise ValueError(f"Unsupported model type for SwiftKV: {hf_config.get('model_type')}")
        hf_config["num_key_value_layers"] = self.config.num_key_value_layers
        hf_config["key_value_group_size"] = self.config.key_value_group_size
        return hf_config

    def _native_class(self, model_config=None):
        if model_config is not None and model_config.get("model_type") == "deepseek_v2":
            return MLASwiftKVForCausalLM
        return SwiftKVForCausalLM

    @staticmethod
    def _init_mla(model) -> None:
        """Queries copied from the teacher branch, every shared latent key/value branch = mean of the teacher
        branches of its group (projections and the latent norm alike), ``norm_swiftkv`` from the first SwiftKV layer."""
        cfg = model.config
        nkv, group = cfg["num_key_value_layers"], max(1, int(cfg.get("key_value_group_size", 1)))
        proj = model.model.swiftkv_kv
        with torch.no_grad():
            proj.norm_swiftkv.weight.copy_(model.model.layers[nkv].input_layernorm.weight)
            proj.norm_swiftkv.weight.requires_grad_(True)
            for layer in model.model.layers[nkv:]:
                attn = layer.self_attn
                for dst, src in zip(attn.q_swiftkv.parameters(), attn.q.parameters()):
                    dst.copy_(src)
                    dst.requires_grad_(True)
            for g, first in enumerate(proj.owner_layers):
                members = model.model.layers[first : first + group]
                for dst in proj.kv_proj[g].parameters():
                    dst.zero_()
                for layer in members:
                    for dst, src in zip(proj.kv_proj[g].parameters(), layer.self_attn.kv.parameters()):
                        dst.add_(src / len(members))
                for dst in proj.kv_proj[g].parameters():
                    dst.requires_grad_(True)

    def post_create_model_callback(self, model):
        cfg = model.config
        nkv, group = cfg["num_key_value_layers"], max(1, int(cfg.get("key_value_group_size", 1)))
        for p in model.parameters():
            p.requires_grad_(False)
        if cfg.get("kv_lora_rank"):
            self._init_mla(model)
            model.activation_checkpointing = not self.config.disable_activation_checkpoint
            return model
        proj = model.model.swiftkv_kv
        hq, hkv, d = cfg["num_attention_heads"], cfg.get("num_key_value_heads") or cfg["num_attention_heads"], cfg.head_dim_
        with torch.no_grad():
            proj.norm_swiftkv.weight.copy_(model.model.layers[nkv].input_layernorm.weight)
            proj.norm_swiftkv.weight.requires_grad_(True)
            for layer in model.model.layers[nkv:]:
                attn = layer.self_attn
                attn.q_proj_swiftkv.weight.copy_(attn.qkv_proj.weight[: hq * d])
                attn.q_proj_swiftkv.weight.requires_grad_(True)
                if attn.q_proj_swiftkv.bias is not None:
                    attn.q_proj_swiftkv.bias.copy_(attn.qkv_proj.bias[: hq * d])
                    attn.q_proj_swiftkv.bias.requires_grad_(True)
            for g, first in enumerate(proj.owner_layers):
                lin = proj.kv_proj[g]
                lin.weight.zero_()
                if lin.bias is not None:
                    lin.bias.zero_()
                members = model.model.layers[first : first + group]
                for layer in members:
                    lin.weight.add_(layer.self_attn.qkv_proj.weight[hq * d :] / len(members))
                    if lin.bias is not None:
                        lin.bias.add_(layer.self_attn.qkv_proj.bias[hq * d :] / len(members))
                lin.weight.requires_grad_(True)
                if lin.bias is not None:
                    lin.bias.requires_grad_(True)
        model.activation_checkpointing = not self.config.disable_activation_checkpoint
        return model


def build_swiftkv_model(checkpoint_dir: str, dtype=torch.bfloat16, device: str = "cuda") -> "SwiftKVForCausalLM":
    """Load an exported SwiftKV checkpoint (HF layout, SwiftKV fields in ``config.json``) for evaluation."""
    from arctictraining_b200.models.arch import load_arch_config
    from arctictraining_b200.models.hf_io import load_pretrained_into

    cfg = load_arch_config(checkpoint_dir)
    with torch.device(device):
        model = (MLASwiftKVForCausalLM if cfg.get("kv_lora_rank") else SwiftKVForCausalLM)(cfg, dtype=dtype)
    load_pretrained_into(model, checkpoint_dir, cfg)
    model.swiftkv(True)
    return model


# ------------------------------------------------------------------------------------------------ tiled KL loss
class _FusedLinearKLFn(torch.autograd.Function):
    """mean over rows of ``weight_t * T^2 * KL(softmax(h_t W^T / T) || softmax(h_s W^T / T))`` with the student
    gradient produced tile by tile inside the forward pass (the vocabulary-sized logits exist for one tile only)."""

    @staticmethod
    def forward(ctx, hs, ht, weight, row_weight, temperature, chunk):
        T = hs.shape[0]
        use_k = _use_kernels(hs) and hs.dtype == torch.bfloat16 and weight.shape[0] % 8 == 0
        dh = torch.empty_like(hs)
        total = torch.zeros((), dtype=torch.float32, device=hs.device)
        inv_rows = 1.0 / T
        for s in range(0, T, chunk):
            e = min(T, s + chunk)
            if use_k:
                tcg = _gemm_ok(hs[s:e], weight)
                zs = gemm(hs[s:e], weight) if tcg else F.linear(hs[s:e], weight)
                zt = gemm(ht[s:e], weight) if tcg else F.linear(ht[s:e], weight)
                rows = _ext.ops().kl_fwd_bwd(zs, zt, row_weight[s:e].contiguous(), temperature, None, True)
                _count()
                total += rows.sum()
                dh[s:e] = (gemm(zs, weight, False, True) if tcg else zs @ weight) * inv_rows
            else:
                zs = F.linear(hs[s:e], weight).float() / temperature
                zt = F.linear(ht[s:e], weight).float() / temperature
                ps, pt = torch.softmax(zs, -1), torch.softmax(zt, -1)
                kl = (pt * (torch.log_softmax(zt, -1) - torch.log_softmax(zs, -1))).sum(-1)
                w = row_weight[s:e]
                total += (kl * w).sum() * temperature**2
                g = ((ps - pt) * (w * temperature).unsqueeze(1)).to(hs.dtype)
                dh[s:e] = (g @ weight) * inv_rows
        ctx.save_for_backward(dh)
        return total * inv_rows

    @staticmethod
    def backward(ctx, gout):
        (dh,) = ctx.saved_tensors
        return dh * gout.to(dh.dtype), None, None, None, None, None


def fused_linear_kl(student_hidden, teacher_hidden, lm_head_weight, mask, temperature: float) -> torch.Tensor:
    hs = student_hidden.reshape(-1, student_hidden.shape[-1]).contiguous()
    ht = teacher_hidden.reshape(-1, teacher_hidden.shape[-1]).contiguous()
    w = mask.reshape(-1).to(torch.float32)
    chunk = max(256, (1 << 29) // (2 * lm_head_weight.shape[0]) // 256 * 256)
    return _FusedLinearKLFn.apply(hs, ht, lm_head_weight, w, float(temperature), chunk)


# ------------------------------------------------------------------------------------------------ trainer
class SwiftKVTrainer(SFTTrainer):
    name = "swiftkv"
    config: SwiftKVTrainerConfig
    model_factory: SwiftKVModelFactory
    checkpoint_engine: Union[DSCheckpointEngine, HFCheckpointEngine]

    def forward(self, batch):
        """Teacher pass without gradient and SwiftKV off, then the student pass from the first SwiftKV layer on
        (the layers before it are frozen and see the same input in both networks)."""
        module = self.model_unwrapped
        inner = module.model
        batch = {k: v for k, v in batch.items() if torch.is_tensor(v)}
        pos = batch.get("position_ids")
        ids = batch["input_ids"]
        if pos is None:
            pos = torch.arange(ids.shape[1], device=ids.device).unsqueeze(0).expand_as(ids)
        ctx = module.build_context(pos)
        nkv = inner.swiftkv_kv.nkv
        with torch.no_grad():
            module.swiftkv(False)
            module.eval()
            t_hidden: List[torch.Tensor] = []
            inner.run_layers(inner.embed_tokens(ids), ctx, 0, t_hidden)
        module.swiftkv(True)
        module.train()
        s_tail: List[torch.Tensor] = []
        start = t_hidden[nkv].detach()
        inner.run_layers(start, ctx, nkv, s_tail)
        s_hidden = t_hidden[:nkv] + s_tail
        return s_hidden, t_hidden

    def compute_logits_loss(self, student_hidden, teacher_hidden, mask):
        return fused_linear_kl(student_hidden, teacher_hidden, self.model_unwrapped.lm_head.weight, mask,
                               self.config.logits_loss_temp)

    def compute_hidden_loss(self, student_hidden, teacher_hidden):
        return F.mse_loss(student_hidden.float(), teacher_hidden.float())

    def loss(self, batch) -> torch.Tensor:
        batch = to_device(batch, self.device)
        batch.pop("packed_sample_seqlens", None)
        s_hidden, t_hidden = self.forward(batch)
        use_sp = self.config.sequence_parallel_size > 1
        labels = batch["shift_labels" if use_sp else "labels"]
        mask = labels != -100
        logits_loss = self.compute_logits_loss(s_hidden[-1], t_hidden[-1], mask)
        layer = self.config.hidden_loss_layer
        hidden_loss = self.compute_hidden_loss(s_hidden[layer], t_hidden[layer])
        loss = logits_loss + self.config.hidden_loss_mult * hidden_loss
        if use_sp:
            loss = self.sp_context.mean(loss)
        return loss
