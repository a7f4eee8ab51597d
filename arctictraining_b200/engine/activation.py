# SPDX-License-Identifier: Apache-2.0
"""Storage for the inputs of checkpointed units, optionally in pinned host memory.

With offload on, the hidden state that enters a layer is copied to a pinned host buffer on a dedicated
stream while the layer computes, and the device copy is dropped as soon as that copy has finished.  In the
backward pass the tensor is brought back on a second stream, and restoring one handle starts the
prefetch of the handle saved just before it, so the copy of layer ``i-1`` overlaps the recompute and
backward of layer ``i``.  The reference does the same job with a synchronous ``.cpu()`` / ``.to(device)``
pair inside a patched checkpoint function (arctic_training/monkey_patches.py:74-80,111-116).
"""

from __future__ import annotations

from typing import Dict
from typing import List
from typing import Optional
from typing import Tuple

import torch


class _Handle:
    def __init__(self, store: "ActivationStore", x: torch.Tensor, offload: bool) -> None:
        self.store = store
        self.device_tensor: Optional[torch.Tensor] = x
        self.host: Optional[torch.Tensor] = None
        self.d2h_done = None
        self.h2d_done = None
        self.prev: Optional["_Handle"] = None
        self.meta = (x.shape, x.dtype)
        if offload:
            self._offload(x)

    def _offload(self, x: torch.Tensor) -> None:
        st = self.store
        host = st.take_host_buffer(x.numel(), x.dtype)
        ready = torch.cuda.Event()
        ready.record()
        with torch.cuda.stream(st.d2h_stream):
            st.d2h_stream.wait_event(ready)
            host.view(x.shape).copy_(x, non_blocking=True)
            self.d2h_done = torch.cuda.Event()
            self.d2h_done.record()
        x.record_stream(st.d2h_stream)
        self.host = host
        self.device_tensor = None  # the caller's references decide when the device copy dies

    def prefetch(self) -> None:
        if self.host is None or self.device_tensor is not None:
            return
        st = self.store
        shape, dtype = self.meta
        with torch.cuda.stream(st.h2d_stream):
            if self.d2h_done is not None:
                st.h2d_stream.wait_event(self.d2h_done)
            dev = torch.empty(shape, dtype=dtype, device=st.device)
            dev.copy_(self.host.view(shape), non_blocking=True)
            self.h2d_done = torch.cuda.Event()
            self.h2d_done.record()
        self.device_tensor = dev

    def restore(self) -> torch.Tensor:
        if self.host is not None:
            self.prefetch()
            torch.cuda.current_stream().wait_event(self.h2d_done)
            self.device_tensor.record_stream(torch.cuda.current_stream())
            if self.prev is not None:
                self.prev.prefetch()
            self.store.give_back_host_buffer(self.host)
            self.host = None
        out = self.device_tensor
        self.device_tensor = None
        self.store.forget(self)
        return out


class ActivationStore:
    def __init__(self, device: torch.device, offload: bool = False) -> None:
        self.device = device
        self.offload = offload and device.type == "cuda"
        self.d2h_stream = torch.cuda.Stream(device=device) if self.offload else None
        self.h2d_stream = torch.cuda.Stream(device=device) if self.offload else None
        self._host_pool: Dict[Tuple[int, torch.dtype], List[torch.Tensor]] = {}
        self._last: Optional[_Handle] = None
        self.bytes_offloaded = 0

    def take_host_buffer(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        pool = self._host_pool.setdefault((numel, dtype), [])
        if pool:
            return pool.pop()
        return torch.empty(numel, dtype=dtype, pin_memory=True)

    def give_back_host_buffer(self, buf: torch.Tensor) -> None:
        self._host_pool.setdefault((buf.numel(), buf.dtype), []).append(buf)

    def save(self, x: torch.Tensor) -> _Handle:
        h = _Handle(self, x.detach(), self.offload)
        if self.offload:
            self.bytes_offloaded += x.numel() * x.element_size()
            h.prev = self._last
            self._last = h
        return h

    def forget(self, h: _Handle) -> None:
        if self._last is h:
            self._last = h.prev
        h.prev = None
