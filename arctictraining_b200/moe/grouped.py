# SPDX-License-Identifier: Apache-2.0
"""Grouped expert MLP over tile-aligned expert segments.

``x`` holds the tokens of all local experts, expert-major, every segment starting at a multiple of 128
rows (padding rows are zero); ``offsets [E+1]`` are the segment starts.  ``w_gate_up [E, 2I, H]`` has
gate/up rows block-interleaved (64/64), ``w_down [E, H, I]``.  On the GPU both GEMMs run on the grouped
tcgen05 kernel (tile -> expert look-up on the device, SwiGLU in the first epilogue); otherwise a loop of
per-expert matmuls — which is what the reference does by default (arctic_training/model/moe/moe.py:54-60).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from ..ops import reference as ref
from ..ops.functional import _use_kernels


def _gated_act(gu: torch.Tensor, act_fn: str) -> torch.Tensor:
    if act_fn == "silu":
        return ref.swiglu_interleaved(gu)
    if act_fn == "silu_alpha":  # gate * sigmoid(1.702 gate) * up
        blocks = gu.reshape(*gu.shape[:-1], gu.shape[-1] // 128, 2, 64)
        g, u = blocks[..., 0, :], blocks[..., 1, :]
        return (g * torch.sigmoid(1.702 * g.float()).to(g.dtype) * u).reshape(*gu.shape[:-1], gu.shape[-1] // 2)
    raise ValueError(f"unsupported expert activation {act_fn!r}")


def grouped_mlp_reference(x: torch.Tensor, offsets: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor,
                          act_fn: str = "silu") -> torch.Tensor:
    E = w_gate_up.shape[0]
    bounds = offsets.tolist()
    out = x.new_zeros(x.shape[0], w_down.shape[1])
    for e in range(E):
        s, t = bounds[e], bounds[e + 1]
        if t > s:
            h = _gated_act(F.linear(x[s:t], w_gate_up[e]), act_fn)
            out[s:t] = F.linear(h, w_down[e])
    return out


def grouped_mlp(x: torch.Tensor, offsets: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor,
                act_fn: str = "silu") -> torch.Tensor:
    if _use_kernels(x) and x.dtype == torch.bfloat16 and act_fn == "silu":  # the fused epilogue is the plain SwiGLU
        from .grouped_cuda import grouped_mlp_cuda

        return grouped_mlp_cuda(x, offsets, w_gate_up, w_down)
    return grouped_mlp_reference(x, offsets, w_gate_up, w_down, act_fn)


def group_gemm_fn(a: torch.Tensor, b: torch.Tensor, rows_cumsum: torch.Tensor) -> torch.Tensor:
    """``C[rows of group g] = A[rows of group g] @ B[g]`` for ``B [G, K, N]`` and inclusive row counts ``rows_cumsum
    [G]`` (group ``g`` owns rows ``rows_cumsum[g-1] : rows_cumsum[g]``).  The stand-alone grouped matmul of the
    reference (arctic_training/model/moe/moe_gemm.py:151-166), differentiable, in the input dtype, ragged tiles
    allowed; the expert MLP of this package does not go through it but through :func:`grouped_mlp`."""
    ends = rows_cumsum.tolist()
    out = a.new_zeros(ends[-1] if ends else 0, b.shape[-1])
    start = 0
    pieces = []
    for g, end in enumerate(ends):
        pieces.append(a[start:end] @ b[g])
        start = end
    return torch.cat(pieces, dim=0) if pieces else out
