# SPDX-License-Identifier: Apache-2.0
"""Grouped expert MLP on the tcgen05 grouped GEMM (``csrc/gemm_sm100.cu``, modes "ragged M" and "ragged K").

The tile -> expert map is resolved on the device from the segment offsets, so neither the forward nor the
backward pass synchronises with the host.
"""

from __future__ import annotations

import torch

from ..ops import _ext
from ..ops.functional import _count

RAGGED_M, RAGGED_K = 1, 2
EPI_STORE, EPI_SWIGLU = 0, 2


def _gg(a, b2d, offsets, mode, b_mn=False, epi=EPI_STORE):
    _count()
    return _ext.ops().gemm_bf16_grouped(a, b2d, offsets, mode, b_mn, epi, None)


class _GroupedLinearFn(torch.autograd.Function):
    """``y[r] = x[r] @ W[g(r)].T`` for tile-aligned expert segments; ``W`` is ``[G, N, K]``."""

    @staticmethod
    def forward(ctx, x, w, offsets):
        G, N, K = w.shape
        ctx.save_for_backward(x, w, offsets)
        return _gg(x, w.view(G * N, K), offsets, RAGGED_M)

    @staticmethod
    def backward(ctx, dy):
        x, w, offsets = ctx.saved_tensors
        G, N, K = w.shape
        dy = dy.contiguous()
        dx = _gg(dy, w.view(G * N, K), offsets, RAGGED_M, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = _gg(dy, x, offsets, RAGGED_K).view(G, N, K) if ctx.needs_input_grad[1] else None
        return dx, dw, None


class _GroupedLinearSwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, offsets):
        G, N, K = w.shape
        if not (ctx.needs_input_grad[0] or ctx.needs_input_grad[1]):
            return _gg(x, w.view(G * N, K), offsets, RAGGED_M, epi=EPI_SWIGLU)
        gu = _gg(x, w.view(G * N, K), offsets, RAGGED_M)
        ctx.save_for_backward(x, w, offsets, gu)
        _count()
        return _ext.ops().swiglu_fwd(gu)

    @staticmethod
    def backward(ctx, dh):
        x, w, offsets, gu = ctx.saved_tensors
        G, N, K = w.shape
        _count()
        dgu = _ext.ops().swiglu_bwd(dh.contiguous(), gu)
        dx = _gg(dgu, w.view(G * N, K), offsets, RAGGED_M, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = _gg(dgu, x, offsets, RAGGED_K).view(G, N, K) if ctx.needs_input_grad[1] else None
        return dx, dw, None


def grouped_mlp_cuda(x: torch.Tensor, offsets: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    assert x.shape[0] % 128 == 0, "expert segments must be padded to 128-row tiles"
    h = _GroupedLinearSwiGLUFn.apply(x.contiguous(), w_gate_up, offsets)
    return _GroupedLinearFn.apply(h, w_down, offsets)
