# SPDX-License-Identifier: Apache-2.0
"""Expert-parallel token exchange over NVLink peer memory.

The sender computes, from the all-gathered per-expert counts, the row that each of its (token, k) pairs occupies in
the owner's expert-major, tile-aligned buffer and stores the token there directly (dispatch); after the experts ran,
the sender pulls its pairs' outputs from the owners and reduces them with the routing weights (combine).  No
send/receive staging, no re-grouping pass on the receiver and no host synchronisation for split sizes, which the
all-to-all formulation needs (arctic_training/model/moe/moe.py:296-371 in the reference).  The backward pass is the
same pair of kernels run the other way.
"""

from __future__ import annotations

import os
from typing import Dict
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import _ext
from ..ops.functional import _count

_EXCHANGES: Dict[int, "PeerMoEExchange"] = {}


class PeerMoEExchange:
    D_SLOT, C_SLOT, BD_SLOT, BC_SLOT, BY_SLOT, N_SLOT = 16, 17, 18, 19, 20, 21

    def __init__(self, group) -> None:
        from ..comm.symm import RotatingBuffers
        from ..comm.symm import SymmetricContext

        self.group = group
        self.symm = SymmetricContext(group)
        self.rank, self.size = self.symm.rank, self.symm.world
        self.rot = RotatingBuffers(self.symm)

    def capacity(self, pairs: int, local_experts: int, align: int) -> int:
        """Rows of the per-rank expert-major buffer: ``ATB200_EP_CAPACITY_FACTOR`` (default 2) times the average
        load, at most the worst case (every pair of every rank on one rank; factor 0 selects it).  A pair that does
        not fit is not written and the communication error word records it (see :func:`check_errors`)."""
        factor = float(os.getenv("ATB200_EP_CAPACITY_FACTOR", "2") or 0)
        rows = self.size * pairs if factor <= 0 else int(min(self.size, factor) * pairs)
        rows += local_experts * (align - 1)
        return (rows + align - 1) // align * align

    def all_counts(self, counts: torch.Tensor) -> torch.Tensor:
        """``[ranks, experts]``: every rank's per-expert pair counts.  Each rank publishes its counts in a symmetric
        slot, a device barrier follows, and every rank reads all peers' slots with the pull kernel (two slots used
        in turn, so that a slot is rewritten only after another barrier has passed): no library collective and no
        host synchronisation on the routing path.  The reference exchanges the counts with an all-to-all
        (arctic_training/model/moe/moe.py:389)."""
        n = counts.numel()
        npad = (n + 3) // 4 * 4  # 16-byte vectors of int32
        if getattr(self, "_counts_buf", None) is None or self._counts_pad != npad:
            torch.cuda.synchronize()
            self._counts_buf = self.symm.alloc(f"moe_counts_{npad}", 2 * npad, torch.int32)
            self._counts_buf.tensor.zero_()
            torch.cuda.synchronize()
            dist.barrier(group=self.group, device_ids=[self.symm.device.index])
            self._counts_pad, self._counts_turn = npad, 0
        turn = self._counts_turn
        self._counts_turn ^= 1
        self._counts_buf.tensor[turn * npad : turn * npad + n].copy_(counts.to(torch.int32).reshape(-1))
        self.symm.barrier(self.N_SLOT)
        out = torch.empty(self.size, npad, dtype=torch.int32, device=counts.device)
        self.symm.all_gather(self._counts_buf, turn * npad, npad, out.view(-1))
        return out[:, :n].to(counts.dtype).contiguous()


def exchange_for(group) -> Optional[PeerMoEExchange]:
    """One exchange per expert-parallel group, or ``None`` when peer memory is not usable."""
    from ..comm.symm import symmetric_memory_available

    key = id(group)
    if key not in _EXCHANGES:
        _EXCHANGES[key] = PeerMoEExchange(group) if symmetric_memory_available(group) else None
    return _EXCHANGES[key]


def check_errors() -> None:
    """Raise if a dispatch ran out of buffer rows or a barrier timed out since the last check (synchronises)."""
    for ex in _EXCHANGES.values():
        if ex is None:
            continue
        code = int(_ext.ops().comm_read_and_clear_error(ex.symm._flags.tensor))
        if code >> 8 == 0x31:
            raise RuntimeError(
                f"expert-parallel dispatch: rank {(code & 0xff) - 1} received more tokens than its buffer holds; "
                "raise ATB200_EP_CAPACITY_FACTOR (0 = worst case)"
            )
        if code:
            from ..exceptions import CommTimeoutError

            raise CommTimeoutError(f"expert-parallel exchange: device-side wait gave up (code {code:#x})")
        break


def _valid_rows(cap: int, seg: torch.Tensor, totals: torch.Tensor) -> torch.Tensor:
    """Mask [cap, 1] of the rows that hold a token (segments are padded to the tile height)."""
    rows = torch.arange(cap, device=seg.device, dtype=torch.int32)
    e = torch.bucketize(rows, seg[1:].contiguous(), right=True).clamp_(max=totals.numel() - 1)
    return (rows < seg[e.long()] + totals[e.long()]).unsqueeze(1)


class _DispatchFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, experts, dest, valid, ex: PeerMoEExchange, cap: int, El: int):
        H = x.shape[1]
        buf, off = ex.rot.take("moe_xin", cap * H)
        for name in ("moe_dxin", "moe_yout", "moe_dyin"):  # buffers of the backward pass: allocate on this thread
            ex.rot.reserve(name, cap * H)
        _count()
        _ext.ops().p2p_moe_dispatch(x.contiguous(), experts, dest, buf.ptrs, off * 2, El, cap, None)
        ex.symm.barrier(ex.D_SLOT)
        ctx.save_for_backward(experts, dest)
        ctx.ex, ctx.cap, ctx.El, ctx.H = ex, cap, El, H
        recv = buf.tensor[off : off + cap * H].view(cap, H)
        return torch.where(valid, recv, torch.zeros((), dtype=recv.dtype, device=recv.device))

    @staticmethod
    def backward(ctx, g):
        experts, dest = ctx.saved_tensors
        ex, cap, El, H = ctx.ex, ctx.cap, ctx.El, ctx.H
        buf, off = ex.rot.take("moe_dxin", cap * H)
        buf.tensor[off : off + cap * H].view(cap, H).copy_(g)
        ex.symm.barrier(ex.BD_SLOT)
        _count()
        dx = _ext.ops().p2p_moe_combine(buf.ptrs, off * 2, experts, dest, None, H, El, cap)
        return dx, None, None, None, None, None, None


class _CombineFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, scores, experts, dest, valid, ex: PeerMoEExchange, cap: int, El: int):
        H = y.shape[1]
        buf, off = ex.rot.take("moe_yout", cap * H)
        buf.tensor[off : off + cap * H].view(cap, H).copy_(y)
        ex.symm.barrier(ex.C_SLOT)
        _count()
        out = _ext.ops().p2p_moe_combine(buf.ptrs, off * 2, experts, dest, scores.contiguous(), H, El, cap)
        ctx.save_for_backward(y, scores, experts, dest, valid)
        ctx.ex, ctx.cap, ctx.El, ctx.H = ex, cap, El, H
        return out

    @staticmethod
    def backward(ctx, dout):
        y, scores, experts, dest, valid = ctx.saved_tensors
        ex, cap, El, H = ctx.ex, ctx.cap, ctx.El, ctx.H
        dout = dout.contiguous()
        # gradient of the routing weights: the owners publish y again (the buffer of the forward pass may have been
        # reused by other layers since), every source takes the dot products for its pairs
        buf, off = ex.rot.take("moe_yout", cap * H)
        buf.tensor[off : off + cap * H].view(cap, H).copy_(y)
        ex.symm.barrier(ex.BY_SLOT)
        _count(2)
        dscores = _ext.ops().p2p_moe_pair_dot(buf.ptrs, off * 2, experts, dest, dout, El, cap)
        # gradient of the expert outputs: score * dout goes to the owner's row of the pair
        gbuf, goff = ex.rot.take("moe_dyin", cap * H)
        _ext.ops().p2p_moe_dispatch(dout, experts, dest, gbuf.ptrs, goff * 2, El, cap, scores.contiguous())
        ex.symm.barrier(ex.BC_SLOT)
        recv = gbuf.tensor[goff : goff + cap * H].view(cap, H)
        dy = torch.where(valid, recv, torch.zeros((), dtype=recv.dtype, device=recv.device))
        return dy, dscores.to(scores.dtype), None, None, None, None, None, None


def peer_expert_forward(x, scores, experts, num_experts: int, ex: PeerMoEExchange, align: int, expert_fn):
    """``out[t] = sum_k scores[t, k] * expert(experts[t, k])(x[t])`` with the experts spread over the group.
    ``expert_fn(tokens [rows, H], segment_offsets [El + 1]) -> [rows, H]`` runs this rank's experts."""
    from . import ops as mops

    P = ex.size
    El = num_experts // P
    T, K = experts.shape
    slots, counts, offsets = mops.assign_slots(experts, num_experts, 1)
    all_counts = ex.all_counts(counts)
    _count()
    dest, seg = _ext.ops().moe_dest_rows(all_counts, experts.contiguous(), slots, offsets, ex.rank, align)
    cap = ex.capacity(T * K, El, align)
    totals = all_counts[:, ex.rank * El : (ex.rank + 1) * El].sum(0).to(torch.int32)
    valid = _valid_rows(cap, seg, totals)
    xin = _DispatchFn.apply(x, experts, dest, valid, ex, cap, El)
    y = expert_fn(xin, seg)
    return _CombineFn.apply(y, scores.float(), experts, dest, valid, ex, cap, El)
