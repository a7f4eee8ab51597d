# SPDX-License-Identifier: Apache-2.0
"""Plain PyTorch implementations of every fused op.

These are the oracle the CUDA kernels are tested against and the code path used on CPU (Gloo runs,
unit tests).  They compute in fp32 internally and return the input dtype.
"""

from __future__ import annotations

import math
from typing import Optional
from typing import Tuple

import torch
import torch.nn.functional as F

IGNORE_INDEX = -100


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    inv = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (xf * inv * weight.float()).to(x.dtype)


def rope_cos_sin(
    position_ids: torch.Tensor, head_dim: int, theta: float, scaling: Optional[dict] = None
) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos/sin tables ``[..., head_dim/2]`` in fp32 for the given positions (rotate-half convention)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=position_ids.device) / head_dim))
    if scaling and scaling.get("rope_type", scaling.get("type")) == "llama3":
        factor = scaling["factor"]
        low, high = scaling["low_freq_factor"], scaling["high_freq_factor"]
        old_len = scaling["original_max_position_embeddings"]
        wavelen = 2 * math.pi / inv_freq
        smooth = ((old_len / wavelen) - low) / (high - low)
        scaled = torch.where(wavelen > old_len / low, inv_freq / factor, inv_freq)
        mid = (1 - smooth) * inv_freq / factor + smooth * inv_freq
        is_mid = (wavelen <= old_len / low) & (wavelen >= old_len / high)
        inv_freq = torch.where(is_mid, mid, scaled)
    amplitude = 1.0
    if scaling and scaling.get("rope_type", scaling.get("type")) == "yarn":
        inv_freq, amplitude = _yarn_inv_freq(inv_freq, head_dim, theta, scaling)
    ang = position_ids.float().unsqueeze(-1) * inv_freq
    if amplitude != 1.0:
        return ang.cos() * amplitude, ang.sin() * amplitude
    return ang.cos(), ang.sin()


def yarn_mscale(factor: float, mscale: float = 1.0) -> float:
    return 1.0 if factor <= 1 else 0.1 * mscale * math.log(factor) + 1.0


def _yarn_inv_freq(inv_freq: torch.Tensor, dim: int, theta: float, scaling: dict):
    """YaRN: frequencies whose wavelength fits ``beta_fast`` times into the original context keep their value, those
    fitting fewer than ``beta_slow`` times are divided by ``factor``, a linear ramp in between; cos/sin are scaled by
    ``mscale(factor, mscale) / mscale(factor, mscale_all_dim)``."""
    factor = float(scaling["factor"])
    orig = float(scaling.get("original_max_position_embeddings") or 4096)
    fast, slow = float(scaling.get("beta_fast") or 32), float(scaling.get("beta_slow") or 1)

    def correction_dim(rotations: float) -> float:
        return dim * math.log(orig / (rotations * 2 * math.pi)) / (2 * math.log(theta))

    low = max(math.floor(correction_dim(fast)), 0)
    high = min(math.ceil(correction_dim(slow)), dim - 1)
    if low == high:
        high += 0.001
    ramp = ((torch.arange(dim // 2, dtype=torch.float32, device=inv_freq.device) - low) / (high - low)).clamp(0, 1)
    keep = 1.0 - ramp
    blended = inv_freq / factor * (1 - keep) + inv_freq * keep
    m, m_all = scaling.get("mscale"), scaling.get("mscale_all_dim")
    amplitude = yarn_mscale(factor, m) / yarn_mscale(factor, m_all) if (m and m_all) else yarn_mscale(factor)
    if scaling.get("attention_factor") is not None:
        amplitude = float(scaling["attention_factor"])
    return blended, float(amplitude)


def rope_apply(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, inverse: bool = False) -> torch.Tensor:
    """Rotate ``x [B, S, H, D]`` with ``cos/sin [B, S, D/2]``: pairs are ``(x[i], x[i + D/2])``."""
    d2 = x.shape[-1] // 2
    xf = x.float()
    x1, x2 = xf[..., :d2], xf[..., d2:]
    c = cos.unsqueeze(-2)
    s = sin.unsqueeze(-2)
    if inverse:
        s = -s
    return torch.cat((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1).to(x.dtype)


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return (F.silu(gate.float()) * up.float()).to(gate.dtype)


GATE_UP_BLOCK = 64


def split_gate_up(gu: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Split a block-interleaved ``[..., 2I]`` tensor (64 gate columns, 64 up columns, ...) into halves."""
    shp = gu.shape
    v = gu.reshape(*shp[:-1], shp[-1] // (2 * GATE_UP_BLOCK), 2, GATE_UP_BLOCK)
    return v[..., 0, :].reshape(*shp[:-1], -1), v[..., 1, :].reshape(*shp[:-1], -1)


def swiglu_interleaved(gu: torch.Tensor) -> torch.Tensor:
    g, u = split_gate_up(gu)
    return swiglu(g, u)


def interleave_gate_up_rows(gate_w: torch.Tensor, up_w: torch.Tensor) -> torch.Tensor:
    """Build the fused ``[2I, H]`` weight whose output columns are block-interleaved (block = 64)."""
    inter, hidden = gate_w.shape
    assert inter % GATE_UP_BLOCK == 0, "intermediate size must be a multiple of 64"
    g = gate_w.reshape(inter // GATE_UP_BLOCK, 1, GATE_UP_BLOCK, hidden)
    u = up_w.reshape(inter // GATE_UP_BLOCK, 1, GATE_UP_BLOCK, hidden)
    return torch.cat((g, u), dim=1).reshape(2 * inter, hidden)


def deinterleave_gate_up_rows(fused: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    two_i, hidden = fused.shape
    v = fused.reshape(two_i // (2 * GATE_UP_BLOCK), 2, GATE_UP_BLOCK, hidden)
    return v[:, 0].reshape(-1, hidden).contiguous(), v[:, 1].reshape(-1, hidden).contiguous()


def segment_ids_from_cu(cu_seqlens: torch.Tensor, total: int) -> torch.Tensor:
    pos = torch.arange(total, device=cu_seqlens.device)
    return torch.bucketize(pos, cu_seqlens[1:], right=True)


def attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    cu_seqlens: Optional[torch.Tensor] = None,
    causal: bool = True,
    scale: Optional[float] = None,
) -> torch.Tensor:
    """Causal GQA attention.  ``q [B,S,Hq,D]``, ``k/v [B,S,Hkv,D]``.  With ``cu_seqlens`` (``B == 1``)
    tokens attend only inside their own packed sample."""
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    qf = q.float().transpose(1, 2)
    kf = k.float().transpose(1, 2).repeat_interleave(Hq // Hkv, dim=1)
    vf = v.float().transpose(1, 2).repeat_interleave(Hq // Hkv, dim=1)
    scores = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    mask = torch.ones(S, S, dtype=torch.bool, device=q.device)
    if causal:
        mask = torch.tril(mask)
    if cu_seqlens is not None:
        seg = segment_ids_from_cu(cu_seqlens, S)
        mask = mask & (seg[:, None] == seg[None, :])
    scores = scores.masked_fill(~mask, float("-inf"))
    out = torch.matmul(torch.softmax(scores, dim=-1), vf)
    return out.transpose(1, 2).to(q.dtype)


def cross_entropy_sum(logits: torch.Tensor, labels: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Sum of token losses (fp32) and the number of labels that are not ``-100``."""
    lf = logits.float()
    loss = F.cross_entropy(lf, labels, ignore_index=IGNORE_INDEX, reduction="sum")
    return loss, (labels != IGNORE_INDEX).sum()


def adamw_step(
    master: torch.Tensor,
    grad: torch.Tensor,
    exp_avg: torch.Tensor,
    exp_avg_sq: torch.Tensor,
    lr: float,
    beta1: float,
    beta2: float,
    eps: float,
    weight_decay: float,
    step: int,
    grad_scale: float = 1.0,
    out_lp: Optional[torch.Tensor] = None,
) -> None:
    """Decoupled-weight-decay Adam on flat tensors, in place; optionally writes a low-precision copy."""
    g = grad.float() * grad_scale
    m = exp_avg.float().mul_(beta1).add_(g, alpha=1 - beta1)
    v = exp_avg_sq.float().mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1 = 1 - beta1**step
    bc2 = 1 - beta2**step
    p = master.float()
    p.mul_(1 - lr * weight_decay)
    denom = (v / bc2).sqrt_().add_(eps)
    p.addcdiv_(m / bc1, denom, value=-lr)
    master.copy_(p)
    exp_avg.copy_(m)
    exp_avg_sq.copy_(v)
    if out_lp is not None:
        out_lp.copy_(p)


def topk_gating(logits: torch.Tensor, top_k: int, normalize: bool) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Softmax over all experts (fp32), top-k (ties → lower index), optional renormalisation.

    Returns ``probs [T,E]`` fp32, ``scores [T,K]`` fp32, ``experts [T,K]`` int64.
    """
    probs = torch.softmax(logits.float(), dim=-1)
    # stable descending sort gives the lower expert index on ties
    order = torch.sort(probs, dim=-1, descending=True, stable=True).indices[:, :top_k]
    scores = torch.gather(probs, 1, order)
    if normalize:
        scores = scores / scores.sum(-1, keepdim=True)
    return probs, scores, order
