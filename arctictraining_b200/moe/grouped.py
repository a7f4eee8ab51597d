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
