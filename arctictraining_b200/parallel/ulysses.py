# SPDX-License-Identifier: Apache-2.0
"""Ulysses sequence parallelism: every rank holds ``S / P`` tokens for everything except core attention,
around which an all-to-all re-shards sequence -> heads (each rank then attends over the full sequence with
``Hq / P`` query heads) and back.

Behaviour parity with what the reference gets from its engine dependency
(arctic_training/trainer/trainer.py:195-202,339-354; arctic_training/trainer/sft_trainer.py:158-164):
* :class:`UlyssesDataLoaderAdapter` — one batch per rank is all-gathered over the SP group and the group
  then works through those batches one after the other (so one dataloader step is ``P`` micro-steps);
  ``labels`` are shifted into ``shift_labels`` *before* the sequence is cut so no token's target lives on
  another rank; every tensor is sliced to this rank's chunk; non-tensor entries pass through.
* KV heads are replicated when there are fewer of them than ranks.
* ``position_ids`` are gathered so that packed-sample boundaries are known for the whole sequence.
* the loss is the token-weighted mean over the group.
"""

from __future__ import annotations

import os
from typing import Any
from typing import Dict
from typing import Iterator
from typing import List
from typing import Optional
from typing import Tuple

import torch
import torch.distributed as dist

from .. import ops

IGNORE_INDEX = -100


class _SeqToHead(torch.autograd.Function):
    """[B, S/P, H, D] -> [B, S, H/P, D] over ``group`` (backward is the inverse exchange)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _seq_to_head(x, group)

    @staticmethod
    def backward(ctx, g):
        return _head_to_seq(g.contiguous(), ctx.group), None


class _HeadToSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _head_to_seq(x, group)

    @staticmethod
    def backward(ctx, g):
        return _seq_to_head(g.contiguous(), ctx.group), None


def _a2a(x: torch.Tensor, group) -> torch.Tensor:
    out = torch.empty_like(x)
    dist.all_to_all_single(out, x, group=group)
    return out


def _seq_to_head(x: torch.Tensor, group) -> torch.Tensor:
    P = dist.get_world_size(group)
    B, S_loc, H, D = x.shape
    send = x.reshape(B, S_loc, P, H // P, D).permute(2, 0, 1, 3, 4).contiguous()  # [P, B, S_loc, H/P, D]
    recv = _a2a(send, group)  # chunk i: sequence chunk of rank i, my head group
    return recv.permute(1, 0, 2, 3, 4).reshape(B, P * S_loc, H // P, D)


def _head_to_seq(x: torch.Tensor, group) -> torch.Tensor:
    P = dist.get_world_size(group)
    B, S, Hl, D = x.shape
    S_loc = S // P
    send = x.reshape(B, P, S_loc, Hl, D).permute(1, 0, 2, 3, 4).contiguous()  # [P, B, S_loc, Hl, D]
    recv = _a2a(send, group)  # chunk j: head group j, my sequence chunk
    return recv.permute(1, 2, 0, 3, 4).reshape(B, S_loc, P * Hl, D)


def _dense_heads(t: torch.Tensor) -> torch.Tensor:
    """[S, H, D] with dense heads and an aligned token stride (views of a fused projection qualify), else a copy."""
    if t.stride(2) == 1 and t.stride(1) == t.shape[2] and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0:
        return t
    return t.contiguous()


class _SumOverGroup(torch.autograd.Function):
    """Forward: all-reduce(sum) so every rank reports the same value; backward: identity, each rank keeps the
    gradient of its own contribution."""

    @staticmethod
    def forward(ctx, x, group):
        y = x.clone()
        dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        return g, None


class _PeerExchange:
    """The two Ulysses exchanges as single kernels over NVLink peer memory (no NCCL call, no permute copies).

    Every exchange owns two symmetric buffers used in turn, and ends with one device-side barrier.  Reusing a
    buffer is safe after two exchanges of the same kind: a rank passes the barrier of exchange n + 1 only after
    every peer has queued, in stream order, its copy out of the buffer of exchange n.  The received data is copied
    out of the symmetric buffer at once, so nothing that autograd saves points into memory peers write to."""

    Q_SLOT, O_SLOT, DO_SLOT, DQ_SLOT, OP_SLOT = 8, 9, 10, 11, 12

    def __init__(self, group) -> None:
        from ..comm.symm import RotatingBuffers
        from ..comm.symm import SymmetricContext

        self.symm = SymmetricContext(group)
        self.rank, self.size = self.symm.rank, self.symm.world
        self._rot = RotatingBuffers(self.symm)

    def _buffer(self, name: str, numel: int):
        return self._rot.take("ulysses_" + name, numel)

    def _reserve(self, name: str, numel: int) -> None:
        self._rot.reserve("ulysses_" + name, numel)

    # ---- q, k, v: sequence-sharded -> head-sharded
    def qkv_seq_to_head(self, q, k, v):
        S_loc, Hq, D = q.shape
        Hkv = k.shape[1]
        P = self.size
        Hlq, Hlkv = Hq // P, (Hkv // P if Hkv >= P else 1)
        W = (Hlq + 2 * Hlkv) * D
        buf, off = self._buffer("qkv", P * S_loc * W)
        self._reserve("dqkv", P * S_loc * W)  # the backward pass publishes d(qkv) of the same size
        ops._ext.ops().p2p_qkv_push(q, k, v, buf.ptrs, off * 2, self.rank)
        self.symm.barrier(self.Q_SLOT)
        return buf.tensor[off : off + P * S_loc * W].view(P * S_loc, Hlq + 2 * Hlkv, D).clone()

    def qkv_grad_head_to_seq(self, g, S_loc: int, Hq: int, Hkv: int, D: int):
        buf, off = self._buffer("dqkv", g.numel())
        buf.tensor[off : off + g.numel()].view_as(g).copy_(g)
        self.symm.barrier(self.DQ_SLOT)
        return ops._ext.ops().p2p_qkv_grad_pull(buf.ptrs, off * 2, g, S_loc, Hq, Hkv, D, self.rank)

    # ---- attention output: head-sharded -> sequence-sharded (and its gradient the other way)
    def head_to_seq(self, y, slot_name: str = "o"):
        S, Hl, D = y.shape
        P = self.size
        buf, off = self._buffer(slot_name, S * Hl * D)
        self._reserve("do", S * Hl * D)
        ops._ext.ops().p2p_seq_to_head(y, buf.ptrs, self.rank, True, off * 2)
        self.symm.barrier(self.O_SLOT)
        return buf.tensor[off : off + S * Hl * D].view(S // P, Hl * P, D).clone()

    def head_to_seq_project(self, y, weight, residual, stage_ctas: Optional[int] = None):
        """``[residual +] head_to_seq(y) @ weight.T`` in one kernel: every rank publishes its head-sharded attention
        output; in the projection GEMM a few CTAs gather this rank's rows from the owners over NVLink into a local
        matrix (each byte crosses the link once) while the other CTAs multiply the row tiles that have arrived.
        Returns ``(out, gathered)``; ``gathered`` is the exchanged activation ``[S / P, H * D]`` (empty with
        ``stage_ctas=0``, where every CTA pair fetches its operand tiles from the owners with TMA instead)."""
        S, Hl, D = y.shape
        P = self.size
        if stage_ctas is None:
            stage_ctas = int(os.getenv("ATB200_STAGE_CTAS", "16"))
        buf, off = self._buffer("o_src", S * Hl * D)
        self._reserve("do", S * Hl * D)
        buf.tensor[off : off + S * Hl * D].view(S, Hl, D).copy_(y)
        self.symm.barrier(self.OP_SLOT)
        ops.functional._count(comm="gemm_bf16_peer_a")
        return ops._ext.ops().gemm_bf16_peer_a(
            buf.ptrs, off * 2, S, Hl * D, self.rank * (S // P), S // P, weight, residual, stage_ctas
        )

    def seq_to_head(self, x, slot_name: str = "do"):
        S_loc, H, D = x.shape
        P = self.size
        buf, off = self._buffer(slot_name, S_loc * H * D)
        ops._ext.ops().p2p_seq_to_head(x, buf.ptrs, self.rank, False, off * 2)
        self.symm.barrier(self.DO_SLOT)
        return buf.tensor[off : off + S_loc * H * D].view(S_loc * P, H // P, D).clone()


class _QKVSeqToHeadPeer(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, ex):
        ctx.ex, ctx.dims = ex, (q.shape[0], q.shape[1], k.shape[1], q.shape[2])
        return ex.qkv_seq_to_head(q, k, v)

    @staticmethod
    def backward(ctx, g):
        S_loc, Hq, Hkv, D = ctx.dims
        d = ctx.ex.qkv_grad_head_to_seq(g.contiguous(), S_loc, Hq, Hkv, D)
        return d[:, :Hq], d[:, Hq : Hq + Hkv], d[:, Hq + Hkv :], None


class _HeadToSeqPeer(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, ex):
        ctx.ex = ex
        return ex.head_to_seq(y.contiguous())

    @staticmethod
    def backward(ctx, g):
        return ctx.ex.seq_to_head(g.contiguous()), None


class _QKVProjectPushPeer(torch.autograd.Function):
    """Fused q|k|v projection whose GEMM epilogue stores every head's columns into the memory of the rank that owns the
    head (sequence -> head exchange without a separate kernel or a local copy of the projection).  Returns the fused
    ``[S, Hlq + 2 Hlkv, D]`` buffer of this rank's heads over the whole sequence, before rotary embedding."""

    @staticmethod
    def forward(ctx, x2, w, ex, Hq, Hkv, D):
        S_loc = x2.shape[0]
        P = ex.size
        Hlq, Hlkv = Hq // P, (Hkv // P if Hkv >= P else 1)
        Wl = (Hlq + 2 * Hlkv) * D
        buf, off = ex._buffer("qkv", P * S_loc * Wl)
        ex._reserve("dqkv", P * S_loc * Wl)
        ops.functional._count(comm="gemm_bf16_push_heads")
        ops._ext.ops().gemm_bf16_push_heads(x2, w, buf.ptrs, off * 2, ex.rank, Hq, Hkv, D)
        ex.symm.barrier(ex.Q_SLOT)
        ctx.save_for_backward(x2, w)
        ctx.ex, ctx.dims = ex, (S_loc, Hq, Hkv, D)
        return buf.tensor[off : off + P * S_loc * Wl].view(P * S_loc, Hlq + 2 * Hlkv, D).clone()

    @staticmethod
    def backward(ctx, g):
        from ..ops.functional import _wgrad
        from ..ops.functional import gemm

        x2, w = ctx.saved_tensors
        S_loc, Hq, Hkv, D = ctx.dims
        d = ctx.ex.qkv_grad_head_to_seq(g.contiguous(), S_loc, Hq, Hkv, D).view(S_loc, -1)
        dx = gemm(d, w, False, True) if ctx.needs_input_grad[0] else None
        dw = _wgrad(d, x2, w) if ctx.needs_input_grad[1] else None
        return dx, dw, None, None, None, None


class _HeadToSeqProjectPeer(torch.autograd.Function):
    """``[r +] head_to_seq(y) W^T`` with the exchange inside the projection GEMM; keeps the gathered activations for
    the weight gradient.  Backward: dA = dOut W goes back to the head owners with the push exchange."""

    @staticmethod
    def forward(ctx, y, w, r2, ex):
        out, gathered = ex.head_to_seq_project(y.contiguous(), w, r2)
        ctx.save_for_backward(gathered, w)
        ctx.ex, ctx.shape = ex, y.shape
        return out

    @staticmethod
    def backward(ctx, dout):
        from ..ops.functional import _wgrad
        from ..ops.functional import gemm

        gathered, w = ctx.saved_tensors
        dout = dout.contiguous()
        S, Hl, D = ctx.shape
        dy = None
        if ctx.needs_input_grad[0]:
            da = gemm(dout, w, False, True)  # [S / P, H * D]
            dy = ctx.ex.seq_to_head(da.view(da.shape[0], -1, D))
        dw = _wgrad(dout, gathered, w) if ctx.needs_input_grad[1] else None
        return dy, dw, (dout if ctx.needs_input_grad[2] else None), None


class UlyssesContext:
    def __init__(self, group, size: int, rank: int, fused: Optional[bool] = None) -> None:
        self.group, self.size, self.rank = group, size, rank
        self.fused = fused  # None: decide on first use (peer memory available and usable shapes)
        self._peer: Optional[_PeerExchange] = None
        self.fused_block_calls = 0  # attention blocks that ran with both exchanges inside GEMMs

    def _peer_exchange(self, q: torch.Tensor) -> Optional[_PeerExchange]:
        if self.fused is False or not q.is_cuda or q.dtype != torch.bfloat16 or q.shape[0] != 1:
            return None
        if self._peer is None:
            from ..comm.symm import symmetric_memory_available

            if not symmetric_memory_available(self.group):
                self.fused = False
                return None
            self._peer = _PeerExchange(self.group)
            self.fused = True
        return self._peer

    # -- attention -------------------------------------------------------------------------------
    def attention(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, ctx: Any) -> torch.Tensor:
        P = self.size
        Hq, Hkv = q.shape[2], k.shape[2]
        if Hq % P != 0:
            raise ValueError(f"query heads ({Hq}) must be divisible by sequence_parallel_size ({P})")
        ex = self._peer_exchange(q) if (Hkv % P == 0 or P % Hkv == 0) and q.shape[-1] % 8 == 0 else None
        if ex is not None:
            D = q.shape[-1]
            Hlq, Hlkv = Hq // P, (Hkv // P if Hkv >= P else 1)
            qkv = _QKVSeqToHeadPeer.apply(_dense_heads(q[0]), _dense_heads(k[0]), _dense_heads(v[0]), ex)
            qf, kf, vf = qkv[None, :, :Hlq], qkv[None, :, Hlq : Hlq + Hlkv], qkv[None, :, Hlq + Hlkv :]
            o = ops.attention(qf, kf, vf, ctx.cu_seqlens, ctx.max_seqlen, True, ctx.attn_impl)
            return _HeadToSeqPeer.apply(o[0], ex)[None]
        if Hkv < P:
            if P % Hkv != 0:
                raise ValueError(f"sequence_parallel_size ({P}) must be a multiple of the KV heads ({Hkv})")
            k = k.repeat_interleave(P // Hkv, dim=2)
            v = v.repeat_interleave(P // Hkv, dim=2)
        elif Hkv % P != 0:
            raise ValueError(f"KV heads ({Hkv}) must be divisible by sequence_parallel_size ({P})")
        qf = _SeqToHead.apply(q.contiguous(), self.group)
        kf = _SeqToHead.apply(k.contiguous(), self.group)
        vf = _SeqToHead.apply(v.contiguous(), self.group)
        o = ops.attention(qf, kf, vf, ctx.cu_seqlens, ctx.max_seqlen, True, ctx.attn_impl)
        return _HeadToSeq.apply(o.contiguous(), self.group)

    def fused_attention_block(self, x, w_qkv, w_out, ctx: Any, Hq: int, Hkv: int, D: int, residual):
        """Whole attention block of a layer with both Ulysses exchanges inside GEMMs: the q|k|v projection pushes its
        output to the head owners from its epilogue, rotary embedding is applied after the exchange (with the positions
        of the whole sequence), and the output projection gathers its operand from the owners.  ``None`` = not
        applicable (caller falls back to separate projection, exchange and attention)."""
        P = self.size
        if os.getenv("ATB200_FUSED_QKV", "1") == "0" or os.getenv("ATB200_FUSED_PROJ", "1") == "0":
            return None
        if x.shape[0] != 1 or x.dtype != torch.bfloat16 or not x.is_cuda or P > 8 or Hq % P or D % 32 or (Hq // P * D) % 64:
            return None
        if not (Hkv % P == 0 or P % Hkv == 0) or w_qkv.dtype != torch.bfloat16 or w_out.dtype != torch.bfloat16:
            return None
        if ctx.rope_fn is None or getattr(self, "global_position_ids", None) is None or x.shape[1] % 8 or x.shape[2] % 8:
            return None
        if residual is not None and (residual.dtype != torch.bfloat16 or not residual.is_contiguous()):
            return None
        if not (w_qkv.is_contiguous() and w_out.is_contiguous() and w_out.shape[0] % 8 == 0):
            return None
        ex = self._peer_exchange(x.view(1, x.shape[1], 1, -1))
        if ex is None:
            return None
        S_loc = x.shape[1]
        if self.global_position_ids.shape[1] != S_loc * P:
            return None
        if "rope_global" not in ctx.extras:
            ctx.extras["rope_global"] = ctx.rope_fn(self.global_position_ids)
        cos, sin = ctx.extras["rope_global"]
        Hlq, Hlkv = Hq // P, (Hkv // P if Hkv >= P else 1)
        self.fused_block_calls += 1
        x2 = x[0] if x[0].is_contiguous() else x[0].contiguous()
        recv = _QKVProjectPushPeer.apply(x2, w_qkv, ex, Hq, Hkv, D)
        q, k, v = ops.rope_qkv(recv.view(1, S_loc * P, (Hlq + 2 * Hlkv) * D), cos, sin, Hlq, Hlkv, D)
        o = ops.attention(q, k, v, ctx.cu_seqlens, ctx.max_seqlen, True, ctx.attn_impl)
        res2 = residual.view(-1, residual.shape[-1]) if residual is not None else None
        return _HeadToSeqProjectPeer.apply(o[0], w_out, res2, ex)[None]

    def attention_project(self, q, k, v, ctx: Any, w_out: torch.Tensor, residual: Optional[torch.Tensor]):
        """Attention followed by the output projection with the head -> sequence exchange done inside the projection
        GEMM.  Returns ``None`` when the fused path does not apply, so that the caller can fall back to
        :meth:`attention` plus a linear layer."""
        P = self.size
        Hq, Hkv, D = q.shape[2], k.shape[2], q.shape[-1]
        if P > 8 or Hq % P or (Hq // P * D) % 64 or w_out.dtype != torch.bfloat16 or os.getenv("ATB200_FUSED_PROJ", "1") == "0":
            return None
        if not ((Hkv % P == 0 or P % Hkv == 0) and D % 8 == 0) or w_out.shape[0] % 8 or not w_out.is_contiguous():
            return None
        if residual is not None and (residual.dtype != torch.bfloat16 or not residual.is_contiguous()):
            return None
        ex = self._peer_exchange(q)
        if ex is None:
            return None
        Hlq, Hlkv = Hq // P, (Hkv // P if Hkv >= P else 1)
        qkv = _QKVSeqToHeadPeer.apply(_dense_heads(q[0]), _dense_heads(k[0]), _dense_heads(v[0]), ex)
        qf, kf, vf = qkv[None, :, :Hlq], qkv[None, :, Hlq : Hlq + Hlkv], qkv[None, :, Hlq + Hlkv :]
        o = ops.attention(qf, kf, vf, ctx.cu_seqlens, ctx.max_seqlen, True, ctx.attn_impl)
        res2 = residual.view(-1, residual.shape[-1]) if residual is not None else None
        return _HeadToSeqProjectPeer.apply(o[0], w_out, res2, ex)[None]

    # -- packed-sample boundaries -------------------------------------------------------------------
    def global_cu_seqlens(self, position_ids: torch.Tensor) -> Tuple[Optional[torch.Tensor], int]:
        from ..models.causal_lm import cu_seqlens_from_position_ids

        parts = [torch.empty_like(position_ids) for _ in range(self.size)]
        dist.all_gather(parts, position_ids.contiguous(), group=self.group)
        full = torch.cat(parts, dim=1)
        self.global_position_ids = full
        cu = cu_seqlens_from_position_ids(full)
        max_len = int((cu[1:] - cu[:-1]).max()) if cu is not None else full.shape[1]
        return cu, max_len

    # -- loss ---------------------------------------------------------------------------------------
    def aggregate_loss(self, loss_sum: torch.Tensor, num_tokens: torch.Tensor) -> torch.Tensor:
        """Token-weighted mean over the group: identical value on every rank, local gradient."""
        n = num_tokens.clone().to(torch.float32)
        dist.all_reduce(n, group=self.group)
        total = _SumOverGroup.apply(loss_sum.float(), self.group)
        return total / n.clamp(min=1.0)

    def mean(self, value: torch.Tensor) -> torch.Tensor:
        return _SumOverGroup.apply(value, self.group) / self.size


def shard_batch_for_rank(batch: Dict[str, Any], sp_rank: int, sp_size: int) -> Dict[str, Any]:
    """``labels`` -> ``shift_labels`` and cut every tensor's sequence dimension to this rank's chunk."""
    out: Dict[str, Any] = {}
    seq_len = None
    for k, v in batch.items():
        if torch.is_tensor(v) and v.dim() >= 2:
            seq_len = v.shape[1]
            break
    if seq_len is not None and seq_len % sp_size != 0:
        raise ValueError(f"sequence length {seq_len} is not divisible by sequence_parallel_size {sp_size}")
    for k, v in batch.items():
        if k == "labels":
            shifted = torch.nn.functional.pad(v[..., 1:], (0, 1), value=IGNORE_INDEX)
            out["shift_labels"] = _chunk(shifted, sp_rank, sp_size)
        elif torch.is_tensor(v) and v.dim() >= 2:
            out[k] = _chunk(v, sp_rank, sp_size)
        else:
            out[k] = v
    return out


def _chunk(t: torch.Tensor, rank: int, size: int) -> torch.Tensor:
    n = t.shape[1] // size
    return t[:, rank * n : (rank + 1) * n].contiguous()


class UlyssesDataLoaderAdapter:
    def __init__(self, dl, sp_rank: int, sp_group, sp_world_size: int, device: torch.device) -> None:
        self.dl, self.sp_rank, self.sp_group, self.sp_world_size, self.device = dl, sp_rank, sp_group, sp_world_size, device

    def __len__(self) -> int:
        return len(self.dl) * self.sp_world_size

    def __getattr__(self, name: str) -> Any:
        return getattr(self.dl, name)

    def __iter__(self) -> Iterator[Dict[str, Any]]:
        for batch in self.dl:
            gathered: List[Any] = [None] * self.sp_world_size
            dist.all_gather_object(gathered, batch, group=self.sp_group)
            for b in gathered:
                yield shard_batch_for_rank(b, self.sp_rank, self.sp_world_size)
