# SPDX-License-Identifier: Apache-2.0
"""Differentiable MoE primitives: gating, deterministic slot assignment, scatter, gather.

CUDA kernels (``csrc/moe.cu``) on the GPU, PyTorch reference on CPU.  All of them are deterministic: slots
inside an expert follow the (token, k) order, so two runs give bit-identical results.
"""

from __future__ import annotations

from typing import Optional
from typing import Tuple

import torch

from ..ops import _ext
from ..ops import reference as ref
from ..ops.functional import _count
from ..ops.functional import _use_kernels


def _load_balance_grad(experts: torch.Tensor, num_experts: int, coeff: float) -> torch.Tensor:
    """``coeff * freq [E]`` with ``freq`` the fraction of (token, k) assignments every expert received: the analytic
    gradient of the load-balancing loss with respect to each token's router probabilities."""
    freq = torch.bincount(experts.reshape(-1).long(), minlength=num_experts).float()
    return freq * (coeff / freq.sum().clamp(min=1))


class _GatingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, top_k, normalize, lb_grad, lb_coeff):
        probs, scores, experts = _ext.ops().moe_topk_gating_fwd(logits.contiguous(), top_k, normalize)
        _count()
        if lb_grad is None and lb_coeff:
            lb_grad = _load_balance_grad(experts, logits.shape[1], lb_coeff)  # from this very routing: one top-k pass
        ctx.save_for_backward(probs, experts, lb_grad if lb_grad is not None else torch.empty(0, device=logits.device))
        ctx.normalize, ctx.has_lb, ctx.in_dtype = normalize, lb_grad is not None, logits.dtype
        ctx.mark_non_differentiable(experts)
        return scores, experts, probs.detach()

    @staticmethod
    def backward(ctx, dscores, _dexperts, _dprobs):
        probs, experts, lb = ctx.saved_tensors
        dlogits = _ext.ops().moe_topk_gating_bwd(dscores.contiguous().float(), probs, experts, lb if ctx.has_lb else None, ctx.normalize)
        _count()
        return dlogits.to(ctx.in_dtype), None, None, None, None


def topk_gating(
    logits: torch.Tensor, top_k: int, normalize: bool, lb_grad: Optional[torch.Tensor] = None, lb_coeff: float = 0.0
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Returns ``scores [T,K]`` (fp32, differentiable), ``experts [T,K]`` (int32) and ``probs [T,E]`` (fp32,
    detached).  ``lb_grad [E]`` is added to d(loss)/d(probs) of every token in the backward pass — the
    analytic gradient of the load-balancing loss; with ``lb_coeff`` instead, that term is ``lb_coeff`` times the
    assignment frequencies of this routing itself (no second routing pass to count them)."""
    if _use_kernels(logits) and logits.shape[1] <= 1024 and top_k <= 32:
        return _GatingFn.apply(logits, top_k, normalize, lb_grad, float(lb_coeff))
    probs = torch.softmax(logits.float(), dim=-1)
    order = torch.sort(probs, dim=-1, descending=True, stable=True).indices[:, :top_k]
    if lb_grad is None and lb_coeff:
        lb_grad = _load_balance_grad(order, logits.shape[1], float(lb_coeff))
    if lb_grad is not None and probs.requires_grad:
        probs.register_hook(lambda g: g + lb_grad.unsqueeze(0))
    scores = torch.gather(probs, 1, order)
    if normalize:
        scores = scores / scores.sum(-1, keepdim=True)
    return scores, order.to(torch.int32), probs.detach()


def assign_slots(experts: torch.Tensor, num_experts: int, align: int = 1) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Expert-major slot of every (token, k) pair; returns ``slots [T,K]``, ``counts [E]`` and the start of
    every expert segment ``offsets [E+1]`` (segments are padded to multiples of ``align`` rows)."""
    if _use_kernels(experts):
        _count(3)
        return _ext.ops().moe_assign_slots(experts.contiguous(), num_experts, align)
    flat = experts.reshape(-1).long()
    counts = torch.bincount(flat, minlength=num_experts)
    padded = (counts + align - 1) // align * align
    offsets = torch.zeros(num_experts + 1, dtype=torch.long, device=experts.device)
    offsets[1:] = torch.cumsum(padded, 0)
    order = torch.sort(flat, stable=True).indices  # pairs grouped by expert, original order kept inside
    rank_in_expert = torch.empty_like(flat)
    starts = torch.cumsum(counts, 0) - counts
    rank_in_expert[order] = torch.arange(flat.numel(), device=flat.device) - starts[flat[order]]
    slots = offsets[flat] + rank_in_expert
    return slots.view_as(experts).to(torch.int32), counts.to(torch.int32), offsets.to(torch.int32)


class _ScatterFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, slots, out_rows):
        ctx.save_for_backward(slots)
        _count()
        return _ext.ops().moe_scatter_fwd(x.contiguous(), slots, out_rows)

    @staticmethod
    def backward(ctx, dout):
        (slots,) = ctx.saved_tensors
        _count()
        return _ext.ops().moe_scatter_bwd(dout.contiguous(), slots), None, None


def scatter_rows(x: torch.Tensor, slots: torch.Tensor, out_rows: int) -> torch.Tensor:
    """``out[slots[t,k]] = x[t]`` into a zero-initialised ``[out_rows, H]`` buffer."""
    if _use_kernels(x) and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0:
        return _ScatterFn.apply(x, slots, out_rows)
    K = slots.shape[1]
    out = x.new_zeros(out_rows, x.shape[1])
    return out.index_copy(0, slots.reshape(-1).long(), x.repeat_interleave(K, dim=0))


class _GatherFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, slots, scores):
        y = y.contiguous()
        scores = scores.contiguous().float()
        ctx.save_for_backward(y, slots, scores)
        _count()
        return _ext.ops().moe_gather_fwd(y, slots, scores)

    @staticmethod
    def backward(ctx, dout):
        y, slots, scores = ctx.saved_tensors
        dy, dscores = _ext.ops().moe_gather_bwd(dout.contiguous(), y, slots, scores)
        _count()
        return dy, None, dscores


def gather_rows(y: torch.Tensor, slots: torch.Tensor, scores: torch.Tensor) -> torch.Tensor:
    """``out[t] = sum_k scores[t,k] * y[slots[t,k]]`` (fp32 accumulation)."""
    if _use_kernels(y) and y.dtype == torch.bfloat16 and y.shape[1] % 8 == 0:
        return _GatherFn.apply(y, slots, scores)
    T, K = slots.shape
    picked = y[slots.reshape(-1).long()].view(T, K, -1).float()
    return (picked * scores.float().unsqueeze(-1)).sum(1).to(y.dtype)
