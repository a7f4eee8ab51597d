# SPDX-License-Identifier: Apache-2.0
"""Ulysses sequence parallelism for models of the ``transformers`` library (architectures this package has no own
implementation of).

Such a model calls an attention function that it looks up by name in the library's registry.  This module registers
one (``"ulysses"``) that turns the rank's slice of the sequence into a slice of the heads before the core attention and
back afterwards:

    q, k, v  [B, H, S/P, D]  --all-to-all-->  [B, S, H/P, D]  --causal attention over the whole sequence-->
    [B, S, H/P, D]  --all-to-all-->  [B, S/P, H, D]

Key/value heads are replicated first when there are fewer of them than ranks.  Packed samples are recognised from the
``position_ids`` the model passes along (gathered over the group once per forward pass, then turned into
``cu_seqlens``), so attention never crosses a sample boundary.  The core is this package's attention op: the tcgen05
kernels for bf16 / head size 128 on the GPU, PyTorch's attention otherwise.  Rotary embeddings need nothing special:
the dataloader adapter slices ``position_ids`` with the tokens, so each rank rotates its tokens by their true positions.

The reference gets the same behaviour from its engine dependency
(``UlyssesSPAttentionHF.register_with_transformers``, arctic_training/trainer/trainer.py:195-202,229-237).
"""

from __future__ import annotations

from typing import Any
from typing import Optional
from typing import Tuple

import torch
import torch.distributed as dist

from .. import ops
from .ulysses import UlyssesContext
from .ulysses import _HeadToSeq
from .ulysses import _SeqToHead

ATTENTION_NAME = "ulysses"


class UlyssesSPAttentionHF:
    """The registered attention function (a callable object that carries the group and a per-pass cache)."""

    def __init__(self, ctx: UlyssesContext, core_attn_implementation: str = "sdpa") -> None:
        self.ctx = ctx
        self.core = "native" if core_attn_implementation in ("native", "flash_attention_2", "flash_attention_3") else "sdpa"
        self._pos_key: Optional[torch.Tensor] = None
        self._pos_val: Tuple[Optional[torch.Tensor], Optional[int]] = (None, None)
        self.calls = 0

    # ------------------------------------------------------------------ packed-sample boundaries
    def _boundaries(self, position_ids: Optional[torch.Tensor], seq_len: int):
        """``(cu_seqlens, max_seqlen)`` of the whole sequence, or ``(None, None)`` when it is one sample per row.
        The same ``position_ids`` tensor reaches every layer of a forward pass: the gather runs once per pass."""
        if position_ids is None:
            return None, None
        if self._pos_key is position_ids:
            return self._pos_val
        pos = position_ids
        if pos.dim() == 3:  # multi-axis rotary positions [3, B, S]: the first axis carries the text positions
            pos = pos[0]
        if pos.shape[-1] != seq_len:
            parts = [torch.empty_like(pos) for _ in range(self.ctx.size)]
            dist.all_gather(parts, pos.contiguous(), group=self.ctx.group)
            pos = torch.cat(parts, dim=-1)
        val: Tuple[Optional[torch.Tensor], Optional[int]] = (None, None)
        if pos.shape[0] == 1:
            starts = torch.nonzero(pos[0] == 0, as_tuple=False).flatten()
            if starts.numel() > 1:
                cu = torch.cat([starts, starts.new_tensor([pos.shape[-1]])]).to(torch.int32)
                if int(cu[0]) != 0:
                    cu = torch.cat([cu.new_zeros(1), cu])
                val = (cu, int((cu[1:] - cu[:-1]).max()))
        self._pos_key, self._pos_val = position_ids, val
        return val

    # ------------------------------------------------------------------ the attention function
    def __call__(self, module: torch.nn.Module, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                 attention_mask: Optional[torch.Tensor] = None, dropout: float = 0.0, scaling: Optional[float] = None,
                 **kwargs: Any):
        if dropout:
            raise ValueError("attention dropout is not supported under sequence parallelism")
        P, group = self.ctx.size, self.ctx.group
        q, k, v = (t.transpose(1, 2).contiguous() for t in (query, key, value))  # [B, S/P, H, D]
        heads_q, heads_kv = q.shape[2], k.shape[2]
        if heads_q % P:
            raise ValueError(f"query heads ({heads_q}) must be divisible by sequence_parallel_size ({P})")
        if heads_kv % P:
            if P % heads_kv:
                raise ValueError(f"key/value heads ({heads_kv}) and sequence_parallel_size ({P}) must divide one another")
            # fewer key/value heads than ranks: every rank needs the head its query heads attend to
            k = k.repeat_interleave(P // heads_kv, dim=2)
            v = v.repeat_interleave(P // heads_kv, dim=2)
        q, k, v = (_SeqToHead.apply(t, group) for t in (q, k, v))  # [B, S, H/P, D]
        cu_seqlens, max_seqlen = self._boundaries(kwargs.get("position_ids"), q.shape[1])
        window = getattr(module, "sliding_window", None)
        out = ops.attention(q, k, v, cu_seqlens=cu_seqlens, max_seqlen=max_seqlen, causal=True, impl=self.core,
                            scale=scaling, window=window)
        self.calls += 1
        return _HeadToSeq.apply(out.contiguous(), group), None  # [B, S/P, H, D], no attention weights


class SequenceParallelUnit:
    """What ``register_with_transformers`` returns: the group accessors user code and engines ask an "mpu" for."""

    def __init__(self, groups: Any) -> None:
        self.groups = groups

    def get_sequence_parallel_group(self):
        return self.groups.sp_group

    def get_sequence_parallel_world_size(self) -> int:
        return self.groups.sp_size

    def get_sequence_parallel_rank(self) -> int:
        return self.groups.sp_rank

    def get_data_parallel_world_size(self) -> int:
        return self.groups.world  # sequence-parallel ranks count as data-parallel ranks for parameter sharding

    def get_data_parallel_rank(self) -> int:
        return self.groups.rank

    def get_data_parallel_group(self):
        return None  # the default (world) group

    def get_model_parallel_world_size(self) -> int:
        return 1

    def get_model_parallel_rank(self) -> int:
        return 0


def register_with_transformers(model_name_or_path: Any, core_attn_implementation: str, sequence_parallel_size: int,
                               micro_batch_size: int = 1, seq_length: Optional[int] = None,
                               seq_length_is_variable: bool = True, **_: Any) -> SequenceParallelUnit:
    """Call shape of the upstream helper (arctic_training/trainer/trainer.py:195-202): build the sequence-parallel
    groups and make models of the transformers library attend through :class:`UlyssesSPAttentionHF`.  Given a model
    object, that model is switched over; given a name, the function also takes the place of
    ``core_attn_implementation`` in the library's registry, so a model created afterwards with that implementation
    uses it.  With ``sequence_parallel_size == 1`` nothing is registered."""
    from .mesh import ParallelGroups

    groups = ParallelGroups(sequence_parallel_size, 1)
    unit = SequenceParallelUnit(groups)
    if sequence_parallel_size <= 1:
        return unit
    ctx = UlyssesContext(groups.sp_group, groups.sp_size, groups.sp_rank)
    if isinstance(model_name_or_path, torch.nn.Module):
        unit.attention = enable_ulysses_for_hf_model(model_name_or_path, ctx, core_attn_implementation)
    else:
        from transformers.masking_utils import AttentionMaskInterface
        from transformers.modeling_utils import AttentionInterface

        unit.attention = UlyssesSPAttentionHF(ctx, core_attn_implementation)
        for name in (ATTENTION_NAME, core_attn_implementation):
            AttentionInterface.register(name, unit.attention)
            AttentionMaskInterface.register(name, _no_mask)
    unit.context = ctx
    return unit


UlyssesSPAttentionHF.register_with_transformers = staticmethod(register_with_transformers)  # type: ignore[attr-defined]


def _no_mask(*args: Any, **kwargs: Any) -> None:
    """Mask builder for the registered name: the attention function masks by itself (causal, per packed sample)."""
    return None


def enable_ulysses_for_hf_model(model: torch.nn.Module, ctx: UlyssesContext, core_attn_implementation: str = "sdpa"
                                ) -> UlyssesSPAttentionHF:
    """Register the attention function and switch ``model`` (a ``transformers`` model) to it."""
    from transformers.masking_utils import AttentionMaskInterface
    from transformers.modeling_utils import AttentionInterface

    fn = UlyssesSPAttentionHF(ctx, core_attn_implementation)
    AttentionInterface.register(ATTENTION_NAME, fn)
    AttentionMaskInterface.register(ATTENTION_NAME, _no_mask)
    configs = [getattr(model, "config", None)]
    configs += [getattr(m, "config", None) for m in model.modules() if getattr(m, "config", None) is not configs[0]]
    seen = set()
    for cfg in configs:
        if cfg is None or id(cfg) in seen:
            continue
        seen.add(id(cfg))
        if hasattr(cfg, "_attn_implementation"):
            cfg._attn_implementation = ATTENTION_NAME
        for sub in ("text_config",):
            inner = getattr(cfg, sub, None)
            if inner is not None and hasattr(inner, "_attn_implementation"):
                inner._attn_implementation = ATTENTION_NAME
    return fn


def chunked_causal_lm_loss_sum(lm_head: torch.nn.Module, hidden: torch.Tensor, shift_labels: torch.Tensor,
                               logits_bytes_per_chunk: int = 1 << 30) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(sum of token losses, number of target tokens)`` of this rank's slice without holding ``[tokens, vocabulary]``
    logits: the slice is cut into chunks of about ``logits_bytes_per_chunk`` of fp32 logits, each chunk's logits are
    recomputed in the backward pass (arctic_training/trainer/sft_trainer.py:101-156 tiles the same way)."""
    from torch.utils.checkpoint import checkpoint

    vocab = getattr(lm_head, "out_features", None) or lm_head.weight.shape[0]
    chunk = max(1, logits_bytes_per_chunk // (4 * vocab))

    def piece(h: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        logits = lm_head(h).float()
        return torch.nn.functional.cross_entropy(logits.flatten(0, -2), y.flatten(), ignore_index=-100, reduction="sum")

    total = hidden.new_zeros((), dtype=torch.float32)
    for h, y in zip(hidden.split(chunk, dim=1), shift_labels.split(chunk, dim=1)):
        if hidden.requires_grad and torch.is_grad_enabled():
            total = total + checkpoint(piece, h, y, use_reentrant=False)
        else:
            total = total + piece(h, y)
    return total, (shift_labels != -100).sum()
