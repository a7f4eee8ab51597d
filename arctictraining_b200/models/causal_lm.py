# SPDX-License-Identifier: Apache-2.0
"""Native decoder-only language model (Llama / Qwen2 / Qwen3 / Qwen3-MoE families).

The forward signature follows the Hugging Face causal-LM convention used by the trainers
(``input_ids``, ``position_ids``, ``labels`` or ``shift_labels``) so recipes and custom trainers written
for the reference (arctic_training/trainer/sft_trainer.py:49-166) keep working, but the modules are this
framework's own and run on its kernels.  The loss is always computed by the tiled fused
linear-cross-entropy op; full-vocabulary logits are only materialised when a caller asks for them.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any
from typing import List
from typing import Optional

import torch
import torch.nn as nn

from .. import ops
from ..ops import reference as ref
from .arch import ArchConfig
from .modules import DecoderLayer
from .modules import ForwardContext
from .modules import RMSNorm


@dataclass
class CausalLMOutput:
    loss: Optional[torch.Tensor] = None
    logits: Optional[torch.Tensor] = None
    hidden_states: Optional[torch.Tensor] = None
    loss_sum: Optional[torch.Tensor] = None
    num_tokens: Optional[torch.Tensor] = None
    aux_loss: Optional[torch.Tensor] = None
    all_hidden_states: Optional[List[torch.Tensor]] = None


def cu_seqlens_from_position_ids(position_ids: torch.Tensor) -> Optional[torch.Tensor]:
    """Packed-sample boundaries: a new sample starts wherever the position id drops back to 0.
    Only defined for a micro-batch of one packed row; returns ``None`` when there is a single sample."""
    if position_ids.dim() != 2 or position_ids.shape[0] != 1:
        return None
    pos = position_ids[0]
    starts = torch.nonzero(pos == 0, as_tuple=False).flatten()
    if starts.numel() <= 1:
        return None
    if starts[0] != 0:
        starts = torch.cat([starts.new_zeros(1), starts])
    return torch.cat([starts, starts.new_tensor([pos.numel()])]).to(torch.int32)


class DecoderModel(nn.Module):
    """Embedding, decoder stack and final norm (the ``model.*`` sub-tree of an HF checkpoint)."""

    def __init__(self, cfg: ArchConfig, dtype=None, device=None) -> None:
        super().__init__()
        self.cfg = cfg
        self.embed_tokens = nn.Embedding(cfg["vocab_size"], cfg["hidden_size"], dtype=dtype, device=device)
        self.layers = nn.ModuleList(
            [self.build_layer(cfg, i, dtype, device) for i in range(cfg["num_hidden_layers"])]
        )
        self.norm = RMSNorm(cfg["hidden_size"], cfg["rms_norm_eps"], dtype=dtype, device=device)

    def build_layer(self, cfg: ArchConfig, idx: int, dtype, device) -> nn.Module:
        return DecoderLayer(cfg, idx, dtype=dtype, device=device)

    def make_context(self, position_ids: torch.Tensor, attn_impl: str, **kw: Any) -> ForwardContext:
        cfg = self.cfg
        def rope_fn(pos: torch.Tensor):
            return ref.rope_cos_sin(pos, cfg.head_dim_, float(cfg.get("rope_theta") or 10000.0), cfg.get("rope_scaling"))

        cos, sin = rope_fn(position_ids)
        return ForwardContext(cos=cos, sin=sin, attn_impl=attn_impl, rope_fn=rope_fn, **kw)

    def forward(
        self,
        input_ids: torch.Tensor,
        position_ids: Optional[torch.Tensor] = None,
        ctx: Optional[ForwardContext] = None,
        output_hidden_states: bool = False,
        **_: Any,
    ):
        B, S = input_ids.shape
        if position_ids is None:
            position_ids = torch.arange(S, device=input_ids.device).unsqueeze(0).expand(B, S)
        if ctx is None:
            cu = cu_seqlens_from_position_ids(position_ids)
            max_len = int((cu[1:] - cu[:-1]).max()) if cu is not None else S
            ctx = self.make_context(position_ids, getattr(self, "attn_impl", "sdpa"), cu_seqlens=cu, max_seqlen=max_len)
        h = self.embed_tokens(input_ids)
        collected = [h] if output_hidden_states else None
        for layer in self.layers:
            h = layer(h, ctx)
            if collected is not None:
                collected.append(h)
        h = self.norm(h)
        if output_hidden_states:
            return h, collected
        return h


class CausalLM(nn.Module):
    decoder_cls = DecoderModel

    def __init__(self, cfg: ArchConfig, dtype=None, device=None) -> None:
        super().__init__()
        self.config = cfg
        self.model = self.decoder_cls(cfg, dtype=dtype, device=device)
        self.lm_head = nn.Linear(cfg["hidden_size"], cfg["vocab_size"], bias=False, dtype=dtype, device=device)
        if cfg.get("tie_word_embeddings"):
            self.lm_head.weight = self.model.embed_tokens.weight
        self.attn_impl = "sdpa"
        self.tiled_mlp = False
        self.sp_context = None  # set by the trainer when sequence parallelism is on
        if cfg.is_moe:
            from ..moe import convert as _moe_convert  # noqa: F401  (registers the HF name converters)

    # -- initialisation ---------------------------------------------------------------------------
    @torch.no_grad()
    def init_weights(self, std: Optional[float] = None, seed: Optional[int] = None) -> None:
        std = std if std is not None else float(self.config.get("initializer_range", 0.02))
        gen = None
        if seed is not None:
            dev = next(self.parameters()).device
            gen = torch.Generator(device=dev)
            gen.manual_seed(seed)
        for name, p in self.named_parameters():
            if p.dim() == 1 and ("norm" in name):
                p.fill_(1.0)
            elif name.endswith("bias"):
                p.zero_()
            elif getattr(p, "_num_experts", 0) and p.shape[0] != p._num_experts:
                # expert-parallel shard: draw the whole stack (one layer at a time) and keep this rank's experts, so
                # that the weights do not depend on the expert-parallel degree
                full = torch.empty((p._num_experts,) + tuple(p.shape[1:]), dtype=p.dtype, device=p.device)
                full.normal_(0.0, std, generator=gen)
                p.copy_(full[p._first_expert : p._first_expert + p.shape[0]])
                del full
            else:
                p.normal_(0.0, std, generator=gen)

    # -- forward ----------------------------------------------------------------------------------
    def build_context(self, position_ids: torch.Tensor, packed_sample_seqlens=None) -> ForwardContext:
        cu = None
        max_len = position_ids.shape[-1]
        sp = self.sp_context
        if sp is not None:
            cu, max_len = sp.global_cu_seqlens(position_ids)
        else:
            cu = cu_seqlens_from_position_ids(position_ids)
            if cu is not None:
                max_len = int((cu[1:] - cu[:-1]).max())
        ctx = self.model.make_context(position_ids, self.attn_impl, cu_seqlens=cu, max_seqlen=max_len)
        ctx.sp = sp
        ctx.tiled_mlp = self.tiled_mlp
        return ctx

    def forward(
        self,
        input_ids: torch.Tensor,
        position_ids: Optional[torch.Tensor] = None,
        labels: Optional[torch.Tensor] = None,
        shift_labels: Optional[torch.Tensor] = None,
        attention_mask: Optional[torch.Tensor] = None,
        use_cache: bool = False,
        return_logits: bool = False,
        output_hidden_states: bool = False,
        hidden_only: bool = False,
        **_: Any,
    ) -> CausalLMOutput:
        B, S = input_ids.shape
        if position_ids is None:
            position_ids = torch.arange(S, device=input_ids.device).unsqueeze(0).expand(B, S)
        ctx = self.build_context(position_ids)
        res = self.model(input_ids, position_ids, ctx, output_hidden_states=output_hidden_states)
        h, all_h = res if output_hidden_states else (res, None)
        out = CausalLMOutput(hidden_states=h, all_hidden_states=all_h)
        if labels is not None and shift_labels is None:
            shift_labels = torch.nn.functional.pad(labels[..., 1:], (0, 1), value=ops.IGNORE_INDEX)
        if shift_labels is not None:
            loss_sum, n = ops.fused_linear_cross_entropy(h, self.lm_head.weight, shift_labels)
            out.loss_sum, out.num_tokens = loss_sum, n
            out.loss = loss_sum / n.clamp(min=1).to(loss_sum.dtype)
            aux = self.collect_aux_loss()
            if aux is not None:
                out.aux_loss = aux
                out.loss = out.loss + aux
        if return_logits or (shift_labels is None and not hidden_only):
            out.logits = ops.linear(h, self.lm_head.weight)
        return out

    def collect_aux_loss(self) -> Optional[torch.Tensor]:
        total = None
        for m in self.modules():
            aux = getattr(m, "pending_aux_loss", None)
            if aux is not None:
                total = aux if total is None else total + aux
                m.pending_aux_loss = None
        return total

    # -- engine hints ----------------------------------------------------------------------------
    def zero_units(self):
        """Sharding/checkpointing granularity for the engine: one unit per decoder layer, one for the
        embedding and one for the final norm + head (merged with the embedding when tied)."""
        units = [("embed", [self.model.embed_tokens], False)]
        for i, layer in enumerate(self.model.layers):
            units.append((f"layer{i}", [layer], True))
        head = [self.model.norm] if self.config.get("tie_word_embeddings") else [self.model.norm, self.lm_head]
        units.append(("head", head, False))
        return units

    def num_parameters(self) -> int:
        seen, n = set(), 0
        for p in self.parameters():
            if id(p) not in seen:
                seen.add(id(p))
                n += getattr(p, "_atb_numel", p.numel())
        return n
