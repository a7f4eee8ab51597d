# SPDX-License-Identifier: Apache-2.0
"""Variable-split all-to-all with autograd (NCCL / Gloo baseline path of the expert-parallel exchange).
Parity: arctic_training/model/moe/alltoall.py:20-59."""

from __future__ import annotations

from typing import List

import torch
import torch.distributed as dist


def _exchange(x: torch.Tensor, send: List[int], recv: List[int], group) -> torch.Tensor:
    out = x.new_empty((int(sum(recv)),) + tuple(x.shape[1:]))
    if dist.get_backend(group) == "gloo":
        outs = list(out.split([int(r) for r in recv]))
        ins = [t.contiguous() for t in x.split([int(s) for s in send])]
        dist.all_to_all(outs, ins, group=group) if hasattr(dist, "all_to_all") and _gloo_has_a2a() else _a2a_by_p2p(outs, ins, group)
        return out
    dist.all_to_all_single(out, x.contiguous(), [int(r) for r in recv], [int(s) for s in send], group=group)
    return out


def _gloo_has_a2a() -> bool:
    return False


def _a2a_by_p2p(outs, ins, group) -> None:
    """All-to-all out of broadcasts-free point-to-point transfers (Gloo has no all_to_all)."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    ranks = dist.get_process_group_ranks(group)
    outs[rank].copy_(ins[rank])
    reqs = []
    for off in range(1, world):
        dst, src = (rank + off) % world, (rank - off) % world
        if ins[dst].numel():
            reqs.append(dist.isend(ins[dst], ranks[dst], group=group))
        if outs[src].numel():
            reqs.append(dist.irecv(outs[src], ranks[src], group=group))
    for r in reqs:
        r.wait()


class _AllToAllV(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, send, recv, group):
        ctx.send, ctx.recv, ctx.group = send, recv, group
        return _exchange(x, send, recv, group)

    @staticmethod
    def backward(ctx, g):
        return _exchange(g.contiguous(), ctx.recv, ctx.send, ctx.group), None, None, None


def all_to_all_v(x: torch.Tensor, send_splits: List[int], recv_splits: List[int], group) -> torch.Tensor:
    """Rows ``[sum(send), ...]`` -> ``[sum(recv), ...]``; chunk ``i`` goes to rank ``i`` of ``group``."""
    return _AllToAllV.apply(x, [int(s) for s in send_splits], [int(r) for r in recv_splits], group)


class _AllToAllEqual(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        out = torch.empty_like(x)
        dist.all_to_all_single(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = torch.empty_like(g)
        dist.all_to_all_single(out, g.contiguous(), group=ctx.group)
        return out, None


def all_to_all_equal(x: torch.Tensor, group) -> torch.Tensor:
    return _AllToAllEqual.apply(x, group)
