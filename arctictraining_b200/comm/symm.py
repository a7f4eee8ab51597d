# SPDX-License-Identifier: Apache-2.0
"""Symmetric (peer-mapped) device memory and the kernels that communicate through it.

Every rank of a node allocates buffers of identical size through ``torch.distributed._symmetric_memory`` and
learns the address at which each peer's buffer is mapped into its own address space (NVLink P2P), plus the
NVSwitch multicast address when the fabric offers one.  The fused kernels of ``csrc/comm_p2p.cu`` take those
address tables and move data with loads and stores issued from the SMs.

Synchronisation between ranks is a flag exchange (:meth:`SymmetricContext.barrier`) whose device-side wait is
bounded: when a peer does not show up within ``timeout_s`` the kernel records an error code and returns;
:meth:`check` turns that into :class:`CommTimeoutError` on the host, and the CUDA context stays usable.
"""

from __future__ import annotations

import os
from typing import Dict

import torch
import torch.distributed as dist

from ..exceptions import CommTimeoutError
from ..ops import _ext
from ..ops.functional import _count

_FLAG_SLOTS = 64
_MAX_PEERS = 16


def symmetric_memory_available(group=None) -> bool:
    """Peer-mapped memory needs CUDA, an initialised NCCL group confined to one node, and the torch API."""
    if not (torch.cuda.is_available() and dist.is_initialized() and dist.get_backend() == "nccl"):
        return False
    if os.getenv("ATB200_FUSED_COMM", "1") == "0":
        return False
    world = dist.get_world_size(group)
    if world < 2 or world > _MAX_PEERS or world > torch.cuda.device_count():
        return False
    import importlib.util

    return importlib.util.find_spec("torch.distributed._symmetric_memory") is not None


class SymmetricBuffer:
    """One symmetric allocation: ``tensor`` is the local part, ``ptrs`` the peers' addresses (CPU int64)."""

    def __init__(self, numel: int, dtype: torch.dtype, group, device: torch.device) -> None:
        import torch.distributed._symmetric_memory as symm_mem

        if group is None:
            group = dist.group.WORLD  # the rendezvous wants an explicit group object or name
        self.tensor = symm_mem.empty(numel, dtype=dtype, device=device)
        self.handle = symm_mem.rendezvous(self.tensor, group)
        self.ptrs = torch.tensor([int(p) for p in self.handle.buffer_ptrs], dtype=torch.int64)
        try:
            self.multicast_ptr = int(self.handle.multicast_ptr) if self.handle.has_multicast_support else 0
        except Exception:
            self.multicast_ptr = 0
        self.rank = self.handle.rank
        self.world = self.handle.world_size

    def peer_view(self, rank: int, numel: int, elem_offset: int = 0) -> torch.Tensor:
        """``numel`` elements of rank ``rank``'s part of this allocation as a tensor on the local device (the peer's
        memory is mapped into this process)."""
        return self.handle.get_buffer(rank, (numel,), self.tensor.dtype, elem_offset)


class SymmetricContext:
    """Address tables, flags and barrier epochs of one process group."""

    def __init__(self, group=None, timeout_s: float = 20.0) -> None:
        _ext.require()
        self.group = group
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.timeout_s = timeout_s
        self.use_nvls = os.getenv("ATB200_NVLS", "0") == "1"
        self._flags = SymmetricBuffer(_FLAG_SLOTS * _MAX_PEERS, torch.int32, group, self.device)
        self._flags.tensor.zero_()
        torch.cuda.synchronize()
        dist.barrier(group=group, device_ids=[self.device.index])
        self._epochs = [0] * _FLAG_SLOTS
        self.buffers: Dict[str, SymmetricBuffer] = {}

    def alloc(self, name: str, numel: int, dtype: torch.dtype) -> SymmetricBuffer:
        buf = SymmetricBuffer(numel, dtype, self.group, self.device)
        self.buffers[name] = buf
        return buf

    def barrier(self, slot: int = 0) -> None:
        """Device-side barrier over the group on the current stream (no host synchronisation)."""
        self._epochs[slot] += 1
        _ext.ops().p2p_barrier(self._flags.ptrs, self.rank, slot, self._epochs[slot], self.timeout_s, self._flags.tensor)
        _count(comm="p2p_barrier")

    def check(self) -> None:
        """Raise if a bounded wait of any communication kernel gave up since the last check (synchronises)."""
        code = int(_ext.ops().comm_read_and_clear_error(self._flags.tensor))
        if code:
            raise CommTimeoutError(
                f"rank {self.rank}: a peer did not reach a device-side barrier within {self.timeout_s}s "
                f"(code {code:#x}, waiting for peer {(code & 0xff) - 1})"
            )

    # ------------------------------------------------------------------ collectives on symmetric buffers
    def all_gather(self, shards: SymmetricBuffer, shard_elem_offset: int, shard_numel: int, out: torch.Tensor) -> None:
        """``out[p * n : (p + 1) * n] = peer p's shards[offset : offset + n]`` (pull over NVLink)."""
        _ext.ops().p2p_all_gather(shards.ptrs, shard_elem_offset * out.element_size(), out, shard_numel, self.rank)
        _count(comm="p2p_all_gather")

    def all_gather_copy_engine(self, shards: SymmetricBuffer, shard_elem_offset: int, shard_numel: int, out: torch.Tensor) -> None:
        """The same gather as :meth:`all_gather`, issued as one asynchronous device-to-device copy per peer: the copies
        run on the copy engines over NVLink and take no SM from the kernels of the compute stream.  Peers are visited
        in a rank-dependent order so that no rank is read by everybody at once."""
        n = shard_numel
        for step in range(self.world):
            r = (self.rank + step) % self.world
            out[r * n : (r + 1) * n].copy_(shards.peer_view(r, n, shard_elem_offset), non_blocking=True)
        from ..ops.functional import COMM_COUNTER  # copies by the driver: counted as communication, not as kernel launches

        COMM_COUNTER["copy_engine_all_gather"] = COMM_COUNTER.get("copy_engine_all_gather", 0) + self.world

    def reduce_scatter_accumulate(self, grads: SymmetricBuffer, elem_offset: int, n: int, acc: torch.Tensor,
                                  scale: float, overwrite: bool, want_sumsq: bool = False) -> torch.Tensor:
        """``acc (+)= scale * sum_p peer_p.grads[offset : offset + n]`` in fp32; optionally returns ||acc||^2."""
        _count(comm="nvls_reduce_scatter" if self.use_nvls and grads.multicast_ptr else "p2p_reduce_scatter")
        if self.use_nvls and grads.multicast_ptr:
            return _ext.ops().nvls_reduce_scatter_accum(grads.multicast_ptr, elem_offset, n, acc, scale, overwrite, want_sumsq)
        return _ext.ops().p2p_reduce_scatter_accum(grads.ptrs, elem_offset, n, acc, scale, overwrite, want_sumsq)


class RotatingBuffers:
    """Named symmetric buffers that are used in two halves in turn.

    A kernel pushes into (or peers pull from) one half, a device-side barrier follows, and the consumer copies the
    data out at once.  Reusing a half is then safe after two exchanges of the same name: a rank passes the barrier
    of exchange n + 1 only after every peer has queued, in stream order, its copy out of the half of exchange n.
    Buffers grow collectively, so every rank of the group must ask for the same sizes in the same order."""

    def __init__(self, ctx: SymmetricContext) -> None:
        self.ctx = ctx
        self._bufs: Dict[str, SymmetricBuffer] = {}
        self._turn: Dict[str, int] = {}

    def reserve(self, name: str, numel: int, dtype: torch.dtype = torch.bfloat16) -> None:
        """Make sure buffer ``name`` can hold two exchanges of ``numel`` elements without taking a turn.  Forward
        passes reserve the buffers of their backward passes, so that no collective allocation happens on an autograd
        worker thread."""
        numel = (numel + 127) // 128 * 128
        buf = self._bufs.get(name)
        if buf is None or buf.tensor.numel() < 2 * numel:
            self._allocate(name, numel, dtype)

    def _allocate(self, name: str, numel: int, dtype: torch.dtype) -> SymmetricBuffer:
        torch.cuda.synchronize()
        buf = self.ctx.alloc(f"{name}_{2 * numel}", 2 * numel, dtype)
        buf.tensor.zero_()
        torch.cuda.synchronize()
        dist.barrier(group=self.ctx.group, device_ids=[self.ctx.device.index])
        self._bufs[name] = buf
        self._turn[name] = 0
        return buf

    def take(self, name: str, numel: int, dtype: torch.dtype = torch.bfloat16):
        """Returns ``(buffer, element offset of the half to use now)``."""
        numel = (numel + 127) // 128 * 128
        buf = self._bufs.get(name)
        if buf is None or buf.tensor.numel() < 2 * numel:
            buf = self._allocate(name, numel, dtype)
        half = buf.tensor.numel() // 2
        turn = self._turn[name]
        self._turn[name] = turn ^ 1
        return buf, turn * half
