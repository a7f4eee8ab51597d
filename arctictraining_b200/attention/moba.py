# SPDX-License-Identifier: Apache-2.0
"""Mixture of Block Attention (MoBA): every query attends to its own key block (causally) plus the ``topk - 1`` earlier
key blocks whose mean key scores highest against the query.

Behaviour parity: projects/moba_attention/moba/moba_naive.py:27-110 (oracle) and moba_efficient.py:31-417 (two varlen
attention calls merged by their log-sum-exp).  ``moba_attn_naive`` materialises the full score matrix and is the test
oracle; ``moba_attn_varlen`` computes block gating once and evaluates attention chunk by chunk with a block mask, which
keeps memory at ``O(chunk x seqlen)`` per head; ``moba_attn_efficient`` is the sparse algorithm of the reference: causal
attention inside the own key block, plus, for every earlier key block, attention of exactly the queries that selected it,
the partial results merged by their log-sum-exp — work and memory ``O(seqlen x topk x chunk)`` instead of
``O(seqlen^2)``.
"""

from __future__ import annotations

import math

import torch


def _gate_mask(q: torch.Tensor, k: torch.Tensor, chunk: int, topk: int) -> torch.Tensor:
    """``[H, S, num_blocks]`` boolean: which key blocks each query may attend to (own block always included)."""
    S, H, D = q.shape
    nblk = math.ceil(S / chunk)
    pad = nblk * chunk - S
    kf = k.float()
    if pad:
        kf = torch.cat([kf, kf.new_zeros(pad, H, D)], dim=0)
        counts = torch.full((nblk,), chunk, device=q.device, dtype=torch.float32)
        counts[-1] = chunk - pad
    else:
        counts = torch.full((nblk,), chunk, device=q.device, dtype=torch.float32)
    means = kf.view(nblk, chunk, H, D).sum(1) / counts.view(-1, 1, 1)  # [N, H, D]
    gate = torch.einsum("shd,nhd->hsn", q.float(), means)
    pos = torch.arange(S, device=q.device)
    blk_of_q = pos // chunk
    blk = torch.arange(nblk, device=q.device)
    future = blk.view(1, -1) >= blk_of_q.view(-1, 1)  # current and later blocks are not scored
    gate = gate.masked_fill(future.unsqueeze(0), float("-inf"))
    own = blk.view(1, -1) == blk_of_q.view(-1, 1)
    gate = gate.masked_fill(own.unsqueeze(0), float("inf"))
    kk = min(topk, nblk)
    idx = torch.topk(gate, k=kk, dim=-1, sorted=False).indices
    mask = torch.zeros_like(gate, dtype=torch.bool).scatter_(-1, idx, True)
    return mask & torch.isfinite(gate).logical_or(own.unsqueeze(0))


def moba_attn_naive(q, k, v, cu_seqlens, max_seqlen: int, moba_chunk_size: int, moba_topk: int) -> torch.Tensor:
    """Brute-force MoBA over packed sequences ``[total, H, D]`` (oracle)."""
    out = torch.zeros_like(q)
    scale = q.shape[-1] ** -0.5
    bounds = cu_seqlens.tolist()
    for s, e in zip(bounds[:-1], bounds[1:]):
        q_, k_, v_ = q[s:e], k[s:e], v[s:e]
        n = e - s
        allowed_blk = _gate_mask(q_, k_, moba_chunk_size, moba_topk)  # [H, n, N]
        allowed = allowed_blk.repeat_interleave(moba_chunk_size, dim=-1)[:, :, :n]
        allowed &= torch.ones(n, n, dtype=torch.bool, device=q.device).tril().unsqueeze(0)
        scores = torch.einsum("xhd,yhd->hxy", q_.float(), k_.float()) * scale
        p = scores.masked_fill(~allowed, float("-inf")).softmax(-1)
        out[s:e] = torch.einsum("hxy,yhd->xhd", p, v_.float()).to(q.dtype)
    return out


def moba_attn_varlen(q, k, v, cu_seqlens, max_seqlen: int, moba_chunk_size: int, moba_topk: int,
                     query_chunk: int = 1024) -> torch.Tensor:
    """Memory-bounded MoBA: same result as :func:`moba_attn_naive`, evaluated ``query_chunk`` queries at a time."""
    out = torch.empty_like(q)
    scale = q.shape[-1] ** -0.5
    bounds = cu_seqlens.tolist()
    for s, e in zip(bounds[:-1], bounds[1:]):
        q_, k_, v_ = q[s:e], k[s:e], v[s:e]
        n = e - s
        allowed_blk = _gate_mask(q_, k_, moba_chunk_size, moba_topk)
        kf, vf = k_.float(), v_.float()
        for a in range(0, n, query_chunk):
            b = min(n, a + query_chunk)
            kv_end = b  # causal: nothing after the last query of the chunk is needed
            allowed = allowed_blk[:, a:b].repeat_interleave(moba_chunk_size, dim=-1)[:, :, :kv_end]
            causal = torch.arange(kv_end, device=q.device).view(1, -1) <= torch.arange(a, b, device=q.device).view(-1, 1)
            scores = torch.einsum("xhd,yhd->hxy", q_[a:b].float(), kf[:kv_end]) * scale
            p = scores.masked_fill(~(allowed & causal.unsqueeze(0)), float("-inf")).softmax(-1)
            out[s + a : s + b] = torch.einsum("hxy,yhd->xhd", p, vf[:kv_end]).to(q.dtype)
    return out


def moba_attn_efficient(q, k, v, cu_seqlens, max_seqlen: int, moba_chunk_size: int, moba_topk: int) -> torch.Tensor:
    """Sparse MoBA (differentiable): same result as :func:`moba_attn_naive`.

    Per sequence: (1) every query attends causally inside its own key block — one batched product over (block, head);
    (2) the gate picks ``topk - 1`` earlier blocks per query and head; per head, the queries that picked a block are
    gathered (padded to the largest group) and attend to that block in full — one batched product over the blocks;
    (3) the partial outputs of a query are merged with weights ``exp(lse_i - lse_total)``.  This is the
    two-call-and-merge scheme of projects/moba_attention/moba/moba_efficient.py:88-417 in the reference, which runs the
    two calls on a variable-length attention library."""
    out = torch.empty_like(q)
    D = q.shape[-1]
    scale = D ** -0.5
    C = moba_chunk_size
    bounds = cu_seqlens.tolist()
    neg = float("-inf")
    for s0, e0 in zip(bounds[:-1], bounds[1:]):
        n = e0 - s0
        H = q.shape[1]
        nblk = math.ceil(n / C)
        pad = nblk * C - n
        q_, k_, v_ = q[s0:e0].float(), k[s0:e0].float(), v[s0:e0].float()
        with torch.no_grad():
            allowed = _gate_mask(q[s0:e0], k[s0:e0], C, moba_topk)  # [H, n, nblk], own block included
        if pad:
            zeros = q_.new_zeros(pad, H, D)
            qp, kp, vp = torch.cat([q_, zeros]), torch.cat([k_, zeros]), torch.cat([v_, zeros])
        else:
            qp, kp, vp = q_, k_, v_
        kb = kp.view(nblk, C, H, D).permute(2, 0, 1, 3)  # [H, nblk, C, D]
        vb = vp.view(nblk, C, H, D).permute(2, 0, 1, 3)
        key_ok = (torch.arange(nblk * C, device=q.device) < n).view(nblk, C)  # padding keys of the last block

        # (1) own block, causal: [H, nblk, C, C]
        qb = qp.view(nblk, C, H, D).permute(2, 0, 1, 3)
        s_own = torch.matmul(qb, kb.transpose(-1, -2)) * scale
        tri = torch.ones(C, C, dtype=torch.bool, device=q.device).tril()
        s_own = s_own.masked_fill(~(tri & key_ok.view(1, nblk, 1, C)), neg)
        lse_own = torch.logsumexp(s_own, dim=-1)                       # [H, nblk, C]
        o_own = torch.matmul(torch.exp(s_own - lse_own.unsqueeze(-1)), vb)  # [H, nblk, C, D]
        lse_own = lse_own.reshape(H, nblk * C)[:, :n]
        o_own = o_own.reshape(H, nblk * C, D)[:, :n]

        # (2) + (3) per head: queries grouped by the earlier block they selected, merged with the own-block part
        own_blk = torch.arange(n, device=q.device) // C
        res = torch.empty(n, H, D, dtype=torch.float32, device=q.device)
        for h in range(H):
            picks = allowed[h] & (own_blk.view(-1, 1) > torch.arange(nblk, device=q.device).view(1, -1))  # [n, nblk]
            qi, bi = torch.nonzero(picks, as_tuple=True)     # pairs (query, selected block), sorted by query
            if qi.numel() == 0:
                res[:, h] = o_own[h]
                continue
            order = torch.sort(bi, stable=True).indices
            qi, bi = qi[order], bi[order]
            counts = torch.bincount(bi, minlength=nblk)
            width = int(counts.max())
            starts = torch.cumsum(counts, 0) - counts
            col = torch.arange(qi.numel(), device=q.device) - starts[bi]   # position of every pair inside its block group
            grid = torch.full((nblk, width), n, dtype=torch.long, device=q.device)  # n = "no query" (a zero row)
            grid[bi, col] = qi
            q_h = torch.cat([q_[:, h], q_.new_zeros(1, D)])[grid]          # [nblk, width, D]
            s_sel = torch.matmul(q_h, kb[h].transpose(-1, -2)) * scale     # [nblk, width, C]
            s_sel = s_sel.masked_fill(~key_ok.view(nblk, 1, C), neg)
            lse_sel = torch.logsumexp(s_sel, dim=-1)                       # [nblk, width]
            o_sel = torch.matmul(torch.exp(s_sel - lse_sel.unsqueeze(-1)), vb[h])  # [nblk, width, D]
            lse_pairs, o_pairs = lse_sel[bi, col], o_sel[bi, col]          # back to the pair list
            mx = lse_own[h].detach().clone().scatter_reduce(0, qi, lse_pairs.detach(), "amax")
            w_own = torch.exp(lse_own[h] - mx)
            w_pairs = torch.exp(lse_pairs - mx[qi])
            denom = w_own.index_add(0, qi, w_pairs)
            num = (o_own[h] * w_own.unsqueeze(-1)).index_add(0, qi, o_pairs * w_pairs.unsqueeze(-1))
            res[:, h] = num / denom.unsqueeze(-1)
        out[s0:e0] = res.to(q.dtype)
    return out


class MoBAContext:
    """Drop-in attention core for the native model: set ``model.sp_context``-style hook via ``install``."""

    def __init__(self, chunk_size: int, topk: int) -> None:
        self.chunk_size, self.topk = chunk_size, topk

    def global_cu_seqlens(self, position_ids: torch.Tensor):
        """Packed-sample boundaries of the batch (there is no sequence sharding here: the local sequence is the global
        one)."""
        from ..models.causal_lm import cu_seqlens_from_position_ids

        cu = cu_seqlens_from_position_ids(position_ids)
        max_len = int((cu[1:] - cu[:-1]).max()) if cu is not None else position_ids.shape[-1]
        return cu, max_len

    def attention(self, q, k, v, ctx) -> torch.Tensor:
        B, S, Hq, D = q.shape
        rep = Hq // k.shape[2]
        outs = []
        for b in range(B):
            cu = ctx.cu_seqlens if (ctx.cu_seqlens is not None and B == 1) else torch.tensor([0, S], device=q.device)
            kb = k[b].repeat_interleave(rep, dim=1)
            vb = v[b].repeat_interleave(rep, dim=1)
            outs.append(moba_attn_efficient(q[b], kb, vb, cu, S, self.chunk_size, self.topk))
        return torch.stack(outs, 0)
