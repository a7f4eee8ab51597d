# SPDX-License-Identifier: Apache-2.0
"""Differentiable front ends of the fused ops.

Each function has one signature and two implementations: the sm_100a kernel from ``csrc`` (used
whenever the tensors live on a GPU) and the PyTorch reference in :mod:`.reference` (CPU, oracle).
"""

from __future__ import annotations

import os
from typing import Optional
from typing import Tuple

import torch
import torch.nn.functional as F

from . import _ext
from . import reference as ref

IGNORE_INDEX = ref.IGNORE_INDEX

# which GEMM serves nn.Linear-shaped work on the GPU: "tcgen05" (this library's kernel) or "cublas"
_GEMM_BACKEND = os.getenv("ATB200_GEMM", "tcgen05")
LAUNCH_COUNTER = {"native": 0}
# launches of this package's communication kernels by kind (peer barrier, pull all-gather, reduce-scatter ...)
COMM_COUNTER: dict = {}


def set_gemm_backend(name: str) -> None:
    global _GEMM_BACKEND
    assert name in ("tcgen05", "cublas")
    _GEMM_BACKEND = name


def gemm_backend() -> str:
    return _GEMM_BACKEND


def _use_kernels(t: torch.Tensor) -> bool:
    return t.is_cuda and _ext.available()


def _count(n: int = 1, comm: str = "") -> None:
    LAUNCH_COUNTER["native"] += n
    if comm:
        COMM_COUNTER[comm] = COMM_COUNTER.get(comm, 0) + n


# ------------------------------------------------------------------------------------------------ RMSNorm
class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1]).contiguous()
        y, rstd = _ext.ops().rmsnorm_fwd(x2, weight.contiguous(), eps)
        _count()
        ctx.save_for_backward(x2, weight, rstd)
        ctx.shp = shp
        return y.view(shp)

    @staticmethod
    def backward(ctx, dy):
        x2, weight, rstd = ctx.saved_tensors
        dx, dw = _ext.ops().rmsnorm_bwd(dy.reshape(x2.shape).contiguous(), x2, weight.contiguous(), rstd)
        _count()
        return dx.view(ctx.shp), dw.to(weight.dtype), None


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    if _use_kernels(x) and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and x.shape[-1] <= 16384:
        return _RMSNormFn.apply(x, weight, eps)
    return ref.rms_norm(x, weight, eps)


# ------------------------------------------------------------------------------------------------ RoPE
class _QKVRopeFn(torch.autograd.Function):
    """Rotates the q and k heads of a fused projection output ``[T, (Hq + 2 Hkv) D]`` in place."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, hq, hkv, d):
        ctx.save_for_backward(cos, sin)
        ctx.dims = (hq, hkv, d)
        T = qkv.shape[0]
        ops = _ext.ops()
        ops.rope_inplace(qkv[:, : hq * d].unflatten(1, (hq, d)), cos, sin, False)
        ops.rope_inplace(qkv[:, hq * d : (hq + hkv) * d].unflatten(1, (hkv, d)), cos, sin, False)
        _count(2)
        ctx.mark_dirty(qkv)
        return qkv

    @staticmethod
    def backward(ctx, dqkv):
        cos, sin = ctx.saved_tensors
        hq, hkv, d = ctx.dims
        dqkv = dqkv.contiguous().clone()
        ops = _ext.ops()
        ops.rope_inplace(dqkv[:, : hq * d].unflatten(1, (hq, d)), cos, sin, True)
        ops.rope_inplace(dqkv[:, hq * d : (hq + hkv) * d].unflatten(1, (hkv, d)), cos, sin, True)
        _count(2)
        return dqkv, None, None, None, None, None


def rope_qkv(
    qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, hq: int, hkv: int, d: int
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Split a fused projection ``[B, S, (Hq + 2 Hkv) D]`` into rotated q, rotated k and v
    (``[B, S, heads, D]`` views).  ``cos/sin`` are ``[B, S, D/2]`` fp32."""
    B, S, _ = qkv.shape
    if _use_kernels(qkv) and qkv.dtype == torch.bfloat16 and d % 16 == 0 and qkv.is_contiguous():
        flat = qkv.view(B * S, -1)
        if not (flat.requires_grad and flat.is_leaf):
            flat = _QKVRopeFn.apply(
                flat, cos.reshape(B * S, d // 2).contiguous(), sin.reshape(B * S, d // 2).contiguous(), hq, hkv, d
            )
            q, k, v = flat.split([hq * d, hkv * d, hkv * d], dim=-1)
            return q.view(B, S, hq, d), k.view(B, S, hkv, d), v.view(B, S, hkv, d)
    q, k, v = qkv.split([hq * d, hkv * d, hkv * d], dim=-1)
    q = ref.rope_apply(q.view(B, S, hq, d), cos, sin)
    k = ref.rope_apply(k.view(B, S, hkv, d), cos, sin)
    return q, k, v.view(B, S, hkv, d)


class _RopeFn(torch.autograd.Function):
    """Out-of-place rotary embedding of one ``[T, heads, D]`` tensor."""

    @staticmethod
    def forward(ctx, x, cos, sin):
        ctx.save_for_backward(cos, sin)
        y = x.contiguous().clone()
        _ext.ops().rope_inplace(y, cos, sin, False)
        _count()
        return y

    @staticmethod
    def backward(ctx, dy):
        cos, sin = ctx.saved_tensors
        dx = dy.contiguous().clone()
        _ext.ops().rope_inplace(dx, cos, sin, True)
        _count()
        return dx, None, None


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotary embedding of ``x [B, S, heads, D]`` with ``cos/sin [B, S, D/2]`` (fp32)."""
    if _use_kernels(x) and x.dtype == torch.bfloat16 and x.shape[-1] % 16 == 0:
        B, S, Hh, D = x.shape
        y = _RopeFn.apply(x.reshape(B * S, Hh, D), cos.reshape(B * S, D // 2).contiguous(), sin.reshape(B * S, D // 2).contiguous())
        return y.view(B, S, Hh, D)
    return ref.rope_apply(x, cos, sin)


# ------------------------------------------------------------------------------------------------ SwiGLU
class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        gu = gu.contiguous()
        ctx.save_for_backward(gu)
        _count()
        return _ext.ops().swiglu_fwd(gu)

    @staticmethod
    def backward(ctx, dout):
        (gu,) = ctx.saved_tensors
        _count()
        return _ext.ops().swiglu_bwd(dout.contiguous(), gu)


def swiglu_interleaved(gu: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` on a block-interleaved gate/up tensor (64 gate columns, 64 up columns, ...)."""
    if _use_kernels(gu) and gu.dtype == torch.bfloat16 and gu.shape[-1] % 128 == 0:
        return _SwiGLUFn.apply(gu)
    return ref.swiglu_interleaved(gu)


# ------------------------------------------------------------------------------------------------ GEMM / linear
def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    a_mn: bool = False,
    b_mn: bool = False,
    epilogue: int = 0,
    out: Optional[torch.Tensor] = None,
    residual: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Raw tcgen05 GEMM (no autograd).  See ``csrc/gemm_sm100.cu`` for the operand conventions.  With
    ``epilogue=1`` the product is added to ``out`` in place, or to ``residual`` into a fresh tensor."""
    _count()
    return _ext.ops().gemm_bf16(a, b, a_mn, b_mn, epilogue, out, 0, residual)


def _gemm_ok(x2: torch.Tensor, w: torch.Tensor) -> bool:
    return (
        _GEMM_BACKEND == "tcgen05"
        and x2.dtype == torch.bfloat16
        and w.dtype == torch.bfloat16
        and x2.shape[-1] % 8 == 0
        and w.shape[0] % 8 == 0
        and x2.shape[0] % 8 == 0
        and x2.data_ptr() % 16 == 0
        and w.data_ptr() % 16 == 0
        and x2.shape[0] > 0
    )


class _LinearFn(torch.autograd.Function):
    """y = x W^T on the tcgen05 kernel; dgrad and wgrad use the same kernel with MN-major operands."""

    @staticmethod
    def forward(ctx, x2, w):
        ctx.save_for_backward(x2, w)
        return gemm(x2, w)

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy, w, False, True)  # [M,N] x [N,K] (B is MN-major)
        if ctx.needs_input_grad[1]:
            dw = _wgrad(dy, x2, w)  # dY^T X : both operands MN-major
        return dx, dw


class _LinearResidualFn(torch.autograd.Function):
    """y = r + x W^T with the addition done in the GEMM epilogue (one pass over the residual stream less)."""

    @staticmethod
    def forward(ctx, x2, w, r2):
        ctx.save_for_backward(x2, w)
        return gemm(x2, w, epilogue=1, residual=r2)

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = gemm(dy, w, False, True) if ctx.needs_input_grad[0] else None
        dw = _wgrad(dy, x2, w) if ctx.needs_input_grad[1] else None
        return dx, dw, (dy if ctx.needs_input_grad[2] else None)


class _LinearSwiGLUFn(torch.autograd.Function):
    """h = swiglu(x W_gu^T).  When no gradient is needed (the first pass of a checkpointed layer, evaluation)
    the activation is applied in the GEMM epilogue and gate/up never reach memory.  When a gradient is
    needed (the recompute pass that directly precedes the backward) gate/up are kept for the backward, which
    saves recomputing the largest GEMM of the layer a second time."""

    @staticmethod
    def forward(ctx, x2, w_gu):
        if not (ctx.needs_input_grad[0] or ctx.needs_input_grad[1]):
            return gemm(x2, w_gu, epilogue=2)
        gu = gemm(x2, w_gu)
        ctx.save_for_backward(x2, w_gu, gu)
        _count()
        return _ext.ops().swiglu_fwd(gu)

    @staticmethod
    def backward(ctx, dh):
        x2, w_gu, gu = ctx.saved_tensors
        _count()
        dgu = _ext.ops().swiglu_bwd(dh.contiguous(), gu)
        del gu
        dx = gemm(dgu, w_gu, False, True) if ctx.needs_input_grad[0] else None
        dw = _wgrad(dgu, x2, w_gu) if ctx.needs_input_grad[1] else None
        return dx, dw


def _wgrad(dy: torch.Tensor, x2: torch.Tensor, w: torch.Tensor) -> Optional[torch.Tensor]:
    """dW = dY^T X.  When the engine has pointed ``w._atb_main_grad`` at the parameter's slice of its flat gradient
    buffer, the GEMM accumulates straight into it and autograd gets no gradient to add (saves writing the
    temporary and a read-modify-write pass over the buffer)."""
    main = getattr(w, "_atb_main_grad", None)
    if main is not None and main.dtype == torch.bfloat16 and main.shape == w.shape and main.is_contiguous():
        if getattr(w, "_atb_grad_fresh", False):
            # first gradient of this step for a buffer the engine did not zero: store instead of accumulate (no fill
            # pass before, no read of the old contents here)
            gemm(dy, x2, True, True, epilogue=0, out=main)
            w._atb_grad_fresh = False
        else:
            gemm(dy, x2, True, True, epilogue=1, out=main)
        return None
    return gemm(dy, x2, True, True)


class _MLPFn(torch.autograd.Function):
    """``[r +] swiglu(x W_gu^T) W_down^T`` keeping only x and the gate/up projections: the activation h is produced
    again by the kernel that back-propagates through it, so a layer that keeps its activations stores one
    ``[tokens, intermediate]`` tensor less."""

    @staticmethod
    def forward(ctx, x2, w_gu, w_down, r2):
        if not any(ctx.needs_input_grad[:3]):
            h = gemm(x2, w_gu, epilogue=2)
        else:
            gu = gemm(x2, w_gu)
            _count()
            h = _ext.ops().swiglu_fwd(gu)
            ctx.save_for_backward(x2, w_gu, w_down, gu)
        if r2 is None:
            return gemm(h, w_down)
        return gemm(h, w_down, epilogue=1, residual=r2)

    @staticmethod
    def backward(ctx, dy):
        x2, w_gu, w_down, gu = ctx.saved_tensors
        dy = dy.contiguous()
        dh = gemm(dy, w_down, False, True)
        _count()
        dgu, h = _ext.ops().swiglu_bwd_recompute(dh, gu)
        del dh, gu
        dw_down = _wgrad(dy, h, w_down) if ctx.needs_input_grad[2] else None
        del h
        dx = gemm(dgu, w_gu, False, True) if ctx.needs_input_grad[0] else None
        dw_gu = _wgrad(dgu, x2, w_gu) if ctx.needs_input_grad[1] else None
        return dx, dw_gu, dw_down, (dy if ctx.needs_input_grad[3] else None)


def mlp_swiglu(
    x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, residual: Optional[torch.Tensor] = None
) -> torch.Tensor:
    """SwiGLU feed-forward block ``[residual +] swiglu(x W_gu^T) W_down^T`` (block-interleaved gate/up weight)."""
    if _use_kernels(x):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        if (
            _gemm_ok(x2, w_gate_up) and w_gate_up.shape[0] % 128 == 0 and w_down.dtype == torch.bfloat16
            and w_down.shape[0] % 8 == 0 and w_down.data_ptr() % 16 == 0
            and (residual is None or (residual.dtype == torch.bfloat16 and residual.is_contiguous()
                                      and residual.data_ptr() % 16 == 0))
        ):
            r2 = residual.view(-1, w_down.shape[0]) if residual is not None else None
            return _MLPFn.apply(x2, w_gate_up, w_down, r2).view(*x.shape[:-1], w_down.shape[0])
    y = linear(linear_swiglu(x, w_gate_up), w_down)
    return y if residual is None else residual + y


def linear(
    x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None
) -> torch.Tensor:
    """``x @ W^T (+ bias) (+ residual)``; on the GPU the residual is added in the GEMM epilogue."""
    if _use_kernels(x):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        if _gemm_ok(x2, weight):
            if residual is not None and bias is None and residual.dtype == torch.bfloat16 and residual.is_contiguous() \
                    and residual.data_ptr() % 16 == 0:
                y = _LinearResidualFn.apply(x2, weight, residual.view(-1, weight.shape[0]))
                return y.view(*x.shape[:-1], weight.shape[0])
            y = _LinearFn.apply(x2, weight)
            if bias is not None:
                y = y + bias
            y = y.view(*x.shape[:-1], weight.shape[0])
            return y if residual is None else residual + y
    y = F.linear(x, weight, bias)
    return y if residual is None else residual + y


def linear_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
    """``swiglu(x @ W_gate_up^T)`` for a block-interleaved fused gate/up weight ``[2I, H]``."""
    if _use_kernels(x):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        if _gemm_ok(x2, w_gate_up) and w_gate_up.shape[0] % 128 == 0:
            h = _LinearSwiGLUFn.apply(x2, w_gate_up)
            return h.view(*x.shape[:-1], w_gate_up.shape[0] // 2)
    return swiglu_interleaved(F.linear(x, w_gate_up))


# ------------------------------------------------------------------------------------------------ attention
class _NativeAttentionFn(torch.autograd.Function):
    """Forward and backward: the package's sm_100a flash-attention kernels.  The forward saves the output and the
    per-row log-sum-exp; the backward recomputes the probabilities from them on the tensor cores.

    ``ATB200_ATTN_BWD=cudnn`` / ``flash`` selects a library backward (cuDNN's fused kernel for unpacked sequences,
    flash-attn's variable-length kernel) for comparisons; the default is the own kernel."""

    @staticmethod
    def forward(ctx, q, k, v, cu, max_seqlen, scale, dense_rows=0):
        # q [T, Hq, D], k / v [T, Hkv, D]; token stride may be that of a fused projection output.
        # dense_rows > 0: the tokens are that many equally long sequences without packing
        T = q.shape[0]
        nseq = cu.numel() - 1
        _count()
        out, lse = _ext.ops().fmha_fwd(q, k, v, cu, T // 128 + nseq, scale)
        ctx.save_for_backward(q, k, v, out, lse, cu)
        ctx.max_seqlen, ctx.scale, ctx.dense_rows = max_seqlen, scale, dense_rows
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse, cu = ctx.saved_tensors
        which = os.getenv("ATB200_ATTN_BWD", "native")
        if which == "native":
            _count(3)
            T = q.shape[0]
            if dout.stride(-1) != 1 or dout.stride(1) != dout.shape[2] or dout.stride(0) % 8 != 0 or dout.data_ptr() % 16:
                dout = dout.contiguous()
            dq, dk, dv = _ext.ops().fmha_bwd(dout, q, k, v, out, lse, cu, T // 128 + cu.numel() - 1, ctx.scale)
            return dq, dk, dv, None, None, None, None
        if which == "cudnn" and ctx.dense_rows and _cudnn_dense_backward_applicable(q, k, v):
            return _cudnn_dense_attention_backward(dout, q, k, v, out, lse, ctx.dense_rows, ctx.scale) + (None,) * 4
        from flash_attn.flash_attn_interface import _flash_attn_varlen_backward

        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        _flash_attn_varlen_backward(
            dout.contiguous(), q, k, v, out, lse, dq, dk, dv, cu, cu, ctx.max_seqlen, ctx.max_seqlen,
            0.0, ctx.scale, True, -1, -1, 0.0, None, False,
        )
        return dq, dk, dv, None, None, None, None


class _RopeAttentionFn(torch.autograd.Function):
    """Rotary embedding + causal attention on a fused projection output ``qkv [T, (Hq + 2 Hkv) * 128]`` in one
    autograd node.  Forward: q and k heads are rotated in place, the attention kernel reads q, k, v as strided views.
    Backward: the attention backward writes dq, dk, dv straight into one tensor laid out like ``qkv`` and the inverse
    rotation runs in place on it, so the gradient of the projection needs no split/concatenate/clone passes."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, cu, max_seqlen, scale, hq, hkv, d, dense_rows):
        T = qkv.shape[0]
        ops = _ext.ops()
        q = qkv[:, : hq * d].unflatten(1, (hq, d))
        k = qkv[:, hq * d : (hq + hkv) * d].unflatten(1, (hkv, d))
        v = qkv[:, (hq + hkv) * d :].unflatten(1, (hkv, d))
        ops.rope_inplace(q, cos, sin, False)
        ops.rope_inplace(k, cos, sin, False)
        out, lse = ops.fmha_fwd(q, k, v, cu, T // 128 + cu.numel() - 1, scale)
        _count(3)
        ctx.save_for_backward(qkv, out, lse, cu, cos, sin)
        ctx.dims, ctx.scale = (hq, hkv, d), scale
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse, cu, cos, sin = ctx.saved_tensors
        hq, hkv, d = ctx.dims
        T = qkv.shape[0]
        ops = _ext.ops()
        q = qkv[:, : hq * d].unflatten(1, (hq, d))
        k = qkv[:, hq * d : (hq + hkv) * d].unflatten(1, (hkv, d))
        v = qkv[:, (hq + hkv) * d :].unflatten(1, (hkv, d))
        if dout.stride(-1) != 1 or dout.stride(1) != dout.shape[2] or dout.stride(0) % 8 != 0 or dout.data_ptr() % 16:
            dout = dout.contiguous()
        dq, dk, dv = ops.fmha_bwd(dout, q, k, v, out, lse, cu, T // 128 + cu.numel() - 1, ctx.scale, True)
        ops.rope_inplace(dq, cos, sin, True)
        ops.rope_inplace(dk, cos, sin, True)
        _count(5)
        # dq, dk, dv are views of one [T, Hq + 2 Hkv, d] tensor: hand that tensor on as the projection's gradient
        width = (hq + 2 * hkv) * d
        assert dq.stride(0) == width and dq.storage_offset() == 0, "fmha_bwd(packed=True) must return views of one buffer"
        dqkv = dq.as_strided((T, width), (width, 1), 0)
        return dqkv, None, None, None, None, None, None, None, None, None


def rope_attention(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, hq: int, hkv: int, d: int,
                   cu_seqlens: Optional[torch.Tensor], max_seqlen: Optional[int], scale: Optional[float] = None
                   ) -> Optional[torch.Tensor]:
    """``attention(rope(q), rope(k), v)`` for a fused projection output ``[B, S, (Hq + 2 Hkv) D]`` on the package's own
    kernels; ``None`` when they do not cover the case (the caller then takes the unfused route).  The projection
    output is overwritten with its rotated version."""
    if not (_use_kernels(qkv) and qkv.dtype == torch.bfloat16 and d == 128 and qkv.is_contiguous() and _ext.available()):
        return None
    if os.getenv("ATB200_ATTN_BWD", "native") != "native" or os.getenv("ATB200_FUSED_ROPE_ATTN", "1") == "0":
        return None
    if qkv.requires_grad and qkv.is_leaf:
        return None
    B, S, _ = qkv.shape
    if cu_seqlens is None or B > 1 or cu_seqlens.numel() <= 2:
        cu = torch.arange(0, (B + 1) * S, S, device=qkv.device, dtype=torch.int32)
        max_seqlen, dense_rows = S, B
    else:
        cu, max_seqlen, dense_rows = cu_seqlens.to(torch.int32), int(max_seqlen or S), 0
    scale = float(scale if scale is not None else d ** -0.5)
    o = _RopeAttentionFn.apply(qkv.view(B * S, -1), cos.reshape(B * S, d // 2).contiguous(), sin.reshape(B * S, d // 2).contiguous(),
                               cu, max_seqlen, scale, hq, hkv, d, dense_rows)
    return o.view(B, S, hq, d)


def _cudnn_dense_backward_applicable(q, k, v) -> bool:
    """Explicit preconditions of the cuDNN comparison path: the operator exists and the [T, H, D] operands can be
    viewed as [rows, S, H, D] (dense heads).  Errors raised by the operator itself are not caught."""
    if getattr(torch.ops.aten, "_scaled_dot_product_cudnn_attention_backward", None) is None:
        return False
    return all(t.stride(-1) == 1 and t.stride(1) == t.shape[2] for t in (q, k, v))


def _cudnn_dense_attention_backward(dout, q, k, v, out, lse, rows: int, scale: float):
    """Backward of causal attention over ``rows`` equally long, unpacked sequences through cuDNN's fused kernel (a
    library kernel kept for comparisons), fed with the output and the log-sum-exp of this package's forward kernel."""
    op = torch.ops.aten._scaled_dot_product_cudnn_attention_backward
    T, Hq, D = q.shape
    S = T // rows
    # placeholders for the (unused, dropout is off) random-number state
    t = torch.zeros(1, 1, 128, D, device=q.device, dtype=q.dtype)
    fo = torch.ops.aten._scaled_dot_product_cudnn_attention(t, t, t, None, True, 0.0, True, False, scale=1.0)
    seed, offset = fo[6], fo[7]

    def bhsd(t):
        return t.as_strided((rows, t.shape[1], S, D), (S * t.stride(0), t.stride(1), t.stride(0), 1), t.storage_offset())

    lse4 = lse.view(Hq, rows, S).permute(1, 0, 2).unsqueeze(-1).contiguous()
    gq, gk, gv = op(bhsd(dout.contiguous()), bhsd(q), bhsd(k), bhsd(v), bhsd(out), lse4, seed, offset, None, None, None,
                    S, S, 0.0, True, scale=scale)
    return (gq.transpose(1, 2).reshape(T, Hq, D), gk.transpose(1, 2).reshape(T, -1, D),
            gv.transpose(1, 2).reshape(T, -1, D))


def _native_attention(q, k, v, cu_seqlens, max_seqlen, scale):
    B, S, Hq, D = q.shape
    dense_rows = 0
    if cu_seqlens is None or B > 1 or cu_seqlens.numel() <= 2:
        cu = torch.arange(0, (B + 1) * S, S, device=q.device, dtype=torch.int32)
        max_seqlen = S
        dense_rows = B
    else:
        cu = cu_seqlens.to(torch.int32)
        max_seqlen = int(max_seqlen or S)
    scale = float(scale if scale is not None else D ** -0.5)
    o = _NativeAttentionFn.apply(
        q.reshape(B * S, Hq, D), k.reshape(B * S, -1, D), v.reshape(B * S, -1, D), cu, max_seqlen, scale, dense_rows
    )
    return o.view(B, S, Hq, D)


def attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    cu_seqlens: Optional[torch.Tensor] = None,
    max_seqlen: Optional[int] = None,
    causal: bool = True,
    impl: str = "sdpa",
    scale: Optional[float] = None,
    window: Optional[int] = None,
) -> torch.Tensor:
    """Causal GQA attention over ``[B, S, H, D]`` tensors; ``cu_seqlens`` marks packed samples (B == 1).  ``window``
    restricts every query to the last ``window`` keys (sliding-window layers of Qwen2 / Mistral); windowed layers run
    on PyTorch's attention with a band mask, sample by sample.

    ``impl == "native"`` runs this package's tcgen05 forward kernel (head_dim 128, causal, bf16) and falls
    back to the flash-attn library for shapes the kernel does not cover."""
    if window is not None and window > 0 and window < q.shape[1]:
        return _windowed_attention(q, k, v, cu_seqlens, scale, int(window))
    if (
        impl == "native" and q.is_cuda and causal and q.dtype == torch.bfloat16 and q.shape[-1] == 128
        and _ext.available()
    ):
        return _native_attention(q, k, v, cu_seqlens, max_seqlen, scale)
    if q.is_cuda and impl in ("flash_attention_2", "flash_attention_3", "native"):
        try:
            from flash_attn import flash_attn_func
            from flash_attn import flash_attn_varlen_func
        except ImportError:  # pragma: no cover
            flash_attn_func = None
        if flash_attn_func is not None and q.dtype in (torch.bfloat16, torch.float16):
            if cu_seqlens is not None and cu_seqlens.numel() > 2:
                B, S, Hq, D = q.shape
                cu = cu_seqlens.to(torch.int32)
                o = flash_attn_varlen_func(
                    q.reshape(B * S, Hq, D), k.reshape(B * S, -1, D), v.reshape(B * S, -1, D),
                    cu, cu, max_seqlen or S, max_seqlen or S, causal=causal, softmax_scale=scale,
                )
                return o.view(B, S, Hq, D)
            return flash_attn_func(q, k, v, causal=causal, softmax_scale=scale)
    if cu_seqlens is None or cu_seqlens.numel() <= 2:
        Hq, Hkv = q.shape[2], k.shape[2]
        o = F.scaled_dot_product_attention(
            q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=causal, scale=scale,
            enable_gqa=(Hq != Hkv),
        )
        return o.transpose(1, 2)
    # packed samples without a varlen kernel: attend sample by sample
    outs = []
    bounds = cu_seqlens.tolist()
    Hq, Hkv = q.shape[2], k.shape[2]
    for s, e in zip(bounds[:-1], bounds[1:]):
        o = F.scaled_dot_product_attention(
            q[:, s:e].transpose(1, 2), k[:, s:e].transpose(1, 2), v[:, s:e].transpose(1, 2), is_causal=causal,
            scale=scale, enable_gqa=(Hq != Hkv),
        )
        outs.append(o.transpose(1, 2))
    return torch.cat(outs, dim=1)


def _windowed_attention(q, k, v, cu_seqlens, scale, window: int) -> torch.Tensor:
    """Causal attention in which query t sees keys ``(t - window, t]`` of its own sample."""
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    bounds = [0, S] if cu_seqlens is None or cu_seqlens.numel() <= 2 else [int(x) for x in cu_seqlens.tolist()]
    outs = []
    for s, e in zip(bounds[:-1], bounds[1:]):
        n = e - s
        pos = torch.arange(n, device=q.device)
        band = (pos.view(1, n) <= pos.view(n, 1)) & (pos.view(1, n) > pos.view(n, 1) - window)
        o = F.scaled_dot_product_attention(
            q[:, s:e].transpose(1, 2), k[:, s:e].transpose(1, 2), v[:, s:e].transpose(1, 2), attn_mask=band, scale=scale,
            enable_gqa=(Hq != Hkv),
        )
        outs.append(o.transpose(1, 2))
    return torch.cat(outs, dim=1)


# ------------------------------------------------------------------------------------------------ fused linear + CE
def _ce_chunk_tokens(vocab: int, budget_bytes: int = 1 << 30) -> int:
    """Tokens per logits tile so that one bf16 tile stays around ``budget_bytes`` (multiple of 256)."""
    t = max(256, budget_bytes // (2 * vocab))
    return int(t // 256 * 256)


class _FusedLinearCEFn(torch.autograd.Function):
    """loss_sum = sum_t CE(h_t W^T, y_t), with dh and dW produced tile by tile inside the forward pass
    so that the ``[tokens, vocab]`` logits never exist as a whole."""

    @staticmethod
    def forward(ctx, h, weight, labels, chunk):
        T, H = h.shape
        use_k = _use_kernels(h) and h.dtype == torch.bfloat16 and weight.shape[0] % 8 == 0
        need_dh, need_dw = h.requires_grad, weight.requires_grad
        dh = torch.empty_like(h) if need_dh else None
        dw = torch.zeros_like(weight) if need_dw else None
        loss_sum = torch.zeros((), dtype=torch.float32, device=h.device)
        for s in range(0, T, chunk):
            e = min(T, s + chunk)
            hc, yc = h[s:e], labels[s:e]
            if use_k:
                tcg = _gemm_ok(hc, weight)
                logits = gemm(hc, weight) if tcg else F.linear(hc, weight)
                loss_rows, _ = _ext.ops().ce_fwd_bwd(logits, yc, None, None, need_dh or need_dw)
                _count()
                loss_sum += loss_rows.sum()
                if need_dh:
                    dh[s:e] = gemm(logits, weight, False, True) if tcg else logits @ weight
                if need_dw:
                    if tcg:
                        gemm(logits, hc, True, True, epilogue=1, out=dw)
                    else:
                        dw.addmm_(logits.t(), hc)
            else:
                logits = F.linear(hc, weight).float()
                lse = torch.logsumexp(logits, dim=-1)
                valid = yc != IGNORE_INDEX
                picked = torch.gather(logits, 1, yc.clamp(min=0).unsqueeze(1)).squeeze(1)
                loss_sum += ((lse - picked) * valid).sum()
                if need_dh or need_dw:
                    g = torch.softmax(logits, dim=-1)
                    g[torch.arange(e - s, device=h.device), yc.clamp(min=0)] -= 1.0
                    g = (g * valid.unsqueeze(1)).to(h.dtype)
                    if need_dh:
                        dh[s:e] = g @ weight
                    if need_dw:
                        dw.addmm_(g.t(), hc)
            del logits
        ctx.save_for_backward(dh, dw)
        return loss_sum

    @staticmethod
    def backward(ctx, gout):
        dh, dw = ctx.saved_tensors
        if dh is not None:
            dh = dh * gout.to(dh.dtype)
        if dw is not None:
            dw = dw * gout.to(dw.dtype)
        return dh, dw, None, None


def fused_linear_cross_entropy(
    hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, chunk_tokens: Optional[int] = None
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Sum of cross-entropy losses of ``hidden @ weight.T`` against ``labels`` (already shifted) and
    the count of labels different from -100.  Logits are produced and consumed one token tile at a time."""
    h = hidden.reshape(-1, hidden.shape[-1])
    y = labels.reshape(-1)
    if not h.is_contiguous():
        h = h.contiguous()
    chunk = chunk_tokens or _ce_chunk_tokens(weight.shape[0])
    loss_sum = _FusedLinearCEFn.apply(h, weight, y, chunk)
    return loss_sum, (y != IGNORE_INDEX).sum()


class _FusedLinearLogProbFn(torch.autograd.Function):
    """Per-token log-probabilities ``log softmax(h W^T)[y]`` (0 where ``y == -100``) without keeping the
    logits; the backward pass recomputes them tile by tile."""

    @staticmethod
    def forward(ctx, h, weight, labels, chunk):
        T = h.shape[0]
        use_k = _use_kernels(h) and h.dtype == torch.bfloat16 and weight.shape[0] % 8 == 0
        out = torch.empty(T, dtype=torch.float32, device=h.device)
        for s in range(0, T, chunk):
            e = min(T, s + chunk)
            hc, yc = h[s:e], labels[s:e]
            if use_k:
                logits = gemm(hc, weight) if _gemm_ok(hc, weight) else F.linear(hc, weight)
                loss_rows, _ = _ext.ops().ce_fwd_bwd(logits, yc, None, None, False)
                _count()
                out[s:e] = -loss_rows
            else:
                logits = F.linear(hc, weight).float()
                lp = torch.log_softmax(logits, dim=-1)
                picked = torch.gather(lp, 1, yc.clamp(min=0).unsqueeze(1)).squeeze(1)
                out[s:e] = picked * (yc != IGNORE_INDEX)
            del logits
        ctx.save_for_backward(h, weight, labels)
        ctx.chunk, ctx.use_k = chunk, use_k
        return out

    @staticmethod
    def backward(ctx, gout):
        h, weight, labels = ctx.saved_tensors
        chunk, use_k = ctx.chunk, ctx.use_k
        T = h.shape[0]
        need_dh, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        dh = torch.empty_like(h) if need_dh else None
        dw = torch.zeros_like(weight) if need_dw else None
        gout = gout.float().contiguous()
        for s in range(0, T, chunk):
            e = min(T, s + chunk)
            hc, yc = h[s:e], labels[s:e]
            if use_k:
                tcg = _gemm_ok(hc, weight)
                logits = gemm(hc, weight) if tcg else F.linear(hc, weight)
                # d logp = -(softmax - onehot) * g
                _ext.ops().ce_fwd_bwd(logits, yc, None, (-gout[s:e]).contiguous(), True)
                _count()
                g = logits
                if need_dh:
                    dh[s:e] = gemm(g, weight, False, True) if tcg else g @ weight
                if need_dw:
                    if tcg:
                        gemm(g, hc, True, True, epilogue=1, out=dw)
                    else:
                        dw.addmm_(g.t(), hc)
            else:
                logits = F.linear(hc, weight).float()
                valid = (yc != IGNORE_INDEX)
                g = -torch.softmax(logits, dim=-1)
                g[torch.arange(e - s, device=h.device), yc.clamp(min=0)] += 1.0
                g = (g * (gout[s:e] * valid).unsqueeze(1)).to(h.dtype)
                if need_dh:
                    dh[s:e] = g @ weight
                if need_dw:
                    dw.addmm_(g.t(), hc)
            del logits
        return dh, dw, None, None


def fused_linear_logprobs(
    hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, chunk_tokens: Optional[int] = None
) -> torch.Tensor:
    """``log p(labels)`` per position for ``hidden @ weight.T`` (same leading shape as ``labels``; 0 at
    ignored positions).  ``labels`` must already be aligned with ``hidden`` (shifted)."""
    h = hidden.reshape(-1, hidden.shape[-1])
    if not h.is_contiguous():
        h = h.contiguous()
    y = labels.reshape(-1)
    chunk = chunk_tokens or _ce_chunk_tokens(weight.shape[0])
    return _FusedLinearLogProbFn.apply(h, weight, y, chunk).view(labels.shape)


# ------------------------------------------------------------------------------------------------ optimizer pieces
def adamw_step(master, grad, exp_avg, exp_avg_sq, lr, beta1, beta2, eps, weight_decay, step, grad_scale=None, out_lp=None):
    """Fused AdamW on flat tensors.  ``grad_scale`` is a python float or a one-element device tensor."""
    if _use_kernels(master) and master.dtype == torch.float32 and grad.dtype in (torch.float32, torch.bfloat16) \
            and exp_avg.dtype == torch.float32 and (out_lp is None or out_lp.dtype == torch.bfloat16):
        gs = grad_scale
        if gs is not None and not torch.is_tensor(gs):
            gs = torch.full((1,), float(gs), dtype=torch.float32, device=master.device) if gs != 1.0 else None
        _ext.ops().adamw_step(master, grad, exp_avg, exp_avg_sq, out_lp, lr, beta1, beta2, eps, weight_decay, step, gs)
        _count()
        return
    gs = float(grad_scale) if grad_scale is not None else 1.0
    if (
        master.device.type == "cpu" and master.dtype == torch.float32 and grad.dtype == torch.float32
        and grad.device.type == "cpu" and exp_avg.dtype == torch.float32 and exp_avg_sq.dtype == torch.float32
        and (out_lp is None or (out_lp.device.type == "cpu" and out_lp.dtype == torch.bfloat16))
        and master.is_contiguous() and grad.is_contiguous()
    ):
        from . import _ext_cpu

        if _ext_cpu.available():
            _ext_cpu.ops().cpu_adamw_step(master, grad, exp_avg, exp_avg_sq, out_lp, lr, beta1, beta2, eps, weight_decay, step, gs)
            return
    ref.adamw_step(master, grad, exp_avg, exp_avg_sq, lr, beta1, beta2, eps, weight_decay, step, gs, out_lp)


def sumsq(x: torch.Tensor) -> torch.Tensor:
    if _use_kernels(x) and x.dtype in (torch.float32, torch.bfloat16) and x.is_contiguous():
        _count()
        return _ext.ops().sumsq(x)
    return x.float().pow(2).sum()


def accumulate_lp_grad(src: torch.Tensor, acc: torch.Tensor, scale: float, overwrite: bool) -> None:
    """``acc (fp32) = [acc +] scale * src`` for a low-precision gradient buffer."""
    if _use_kernels(src) and src.dtype == torch.bfloat16 and acc.dtype == torch.float32 \
            and src.data_ptr() % 16 == 0 and acc.data_ptr() % 16 == 0:
        _ext.ops().accum_bf16(src, acc, scale, overwrite)
        _count()
        return
    if overwrite:
        acc.copy_(src.to(acc.dtype) * scale)
    else:
        acc.add_(src.to(acc.dtype), alpha=scale)
