# SPDX-License-Identifier: Apache-2.0
"""Contrastive losses for embedding models: InfoNCE with many-to-many relevance labels, and the one-size
Matryoshka variant.  Behaviour parity: projects/arctic_embed/src/arctic_embed/core/losses.py:36-207.

``relations[i, j]`` is 1 for a positive query/document pair, -1 for a labelled negative, 0 for "no label"
(excluded from the softmax).  A query with several positives contributes one softmax row per positive, in which
the other positives of that query are masked out.  The forward pass works on row sub-batches and the backward
pass is written by hand, so only one ``[rows, documents]`` matrix is alive at a time.
"""

from __future__ import annotations

from typing import Optional
from typing import Tuple

import torch
import torch.nn.functional as F
from torch import Tensor

_MASKED = -1e12


class _InfoNCE(torch.autograd.Function):
    SUB_BATCH = 1024

    @staticmethod
    def forward(ctx, scores: Tensor, relations: Tensor, temperature: float) -> Tensor:
        pos_row, pos_col = torch.nonzero(relations == 1, as_tuple=True)
        n_rows = pos_row.numel()
        if n_rows == 0:
            raise ValueError("InfoNCE needs at least one positive pair")
        expanded = n_rows != scores.size(0) or not torch.equal(pos_row, torch.arange(n_rows, device=pos_row.device))
        if expanded:
            rel = relations.clone()
            rel[pos_row, pos_col] = 0  # other positives of the same query never act as negatives
            rel = rel[pos_row]
            rel[torch.arange(n_rows, device=rel.device), pos_col] = 1
            sc = scores[pos_row]
        else:
            rel, sc = relations, scores
        logits = sc.float().masked_fill(rel == 0, _MASKED) / temperature
        total = logits.new_zeros(())
        for s in range(0, n_rows, _InfoNCE.SUB_BATCH):
            total = total + F.cross_entropy(logits[s : s + _InfoNCE.SUB_BATCH], pos_col[s : s + _InfoNCE.SUB_BATCH], reduction="sum")
        ctx.save_for_backward(pos_row, pos_col, logits)
        ctx.temperature, ctx.expanded, ctx.shape, ctx.dtype = temperature, expanded, scores.shape, scores.dtype
        return total / n_rows

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad_output: Tensor):
        pos_row, pos_col, logits = ctx.saved_tensors
        n_rows = logits.size(0)
        g = torch.softmax(logits, dim=-1)
        g[torch.arange(n_rows, device=g.device), pos_col] -= 1.0
        g = g * (grad_output / n_rows / ctx.temperature)
        if ctx.expanded:
            out = torch.zeros(ctx.shape, dtype=g.dtype, device=g.device)
            out.index_add_(0, pos_row, g)
            g = out
        return g.to(ctx.dtype), None, None


def info_nce_loss(scores: Tensor, relations: Tensor, temperature: float = 0.01) -> Tensor:
    """Mean over positive pairs of ``-log softmax(scores / T)[positive]`` over the labelled documents."""
    return _InfoNCE.apply(scores, relations, temperature)


def _truncated_infonce(q: Tensor, d: Tensor, relations: Tensor, dim: int, temperature: float) -> Tensor:
    qn = F.normalize(q[:, :dim].float(), dim=1)
    dn = F.normalize(d[:, :dim].float(), dim=1)
    return info_nce_loss(qn @ dn.t(), relations, temperature)


def one_size_truncated_mrl_info_nce_loss(
    query_embeddings: Tensor, document_embeddings: Tensor, relations: Tensor, truncated_dimension: Optional[int] = None,
    mrl_weight: float = 0.5, temperature: float = 0.01,
) -> Tuple[Tensor, Tensor, Optional[Tensor]]:
    """``(1 - w) * InfoNCE(full dim) + w * InfoNCE(first truncated_dimension dims)``; returns (loss, full, truncated)."""
    assert 0 < mrl_weight < 1
    full = query_embeddings.size(1)
    assert truncated_dimension is None or 0 < truncated_dimension < full
    loss_full = _truncated_infonce(query_embeddings, document_embeddings, relations, full, temperature)
    if truncated_dimension is None:
        return loss_full, loss_full, None
    loss_trunc = _truncated_infonce(query_embeddings, document_embeddings, relations, truncated_dimension, temperature)
    return (1 - mrl_weight) * loss_full + mrl_weight * loss_trunc, loss_full, loss_trunc
