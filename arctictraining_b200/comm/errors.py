# SPDX-License-Identifier: Apache-2.0
"""Turns the per-device error words of the CUDA kernels into Python exceptions.

Every device-side wait of this library is bounded: a kernel that gives up records a code and returns, so the CUDA
context stays usable, but what it was producing is incomplete.  Two words exist per device: one for the compute
kernels (GEMM and attention barrier waits), one for the communication kernels (peer barriers, staging waits,
expert-parallel buffer overflow).  The training engine reads both before every optimizer step and before every
checkpoint, so that an update is never applied to, and a checkpoint never written from, partial results.
"""

from __future__ import annotations

from typing import Tuple

import torch

from ..exceptions import CommTimeoutError
from ..exceptions import KernelWaitError

EP_OVERFLOW = 0x31


def read_error_words(like: torch.Tensor) -> Tuple[int, int]:
    """``(compute word, communication word)`` of ``like``'s device, both cleared (synchronises the device)."""
    from ..ops import _ext

    if not like.is_cuda or not _ext.available():
        return 0, 0
    ops = _ext.ops()
    return int(ops.read_and_clear_error_flag(like)), int(ops.comm_read_and_clear_error(like))


def raise_for_error_words(kernel_code: int, comm_code: int, rank: int = 0) -> None:
    if comm_code:
        if comm_code >> 8 == EP_OVERFLOW:
            raise RuntimeError(
                f"expert-parallel dispatch: rank {(comm_code & 0xff) - 1} received more tokens than its buffer holds; "
                "raise ATB200_EP_CAPACITY_FACTOR (0 = worst case)"
            )
        raise CommTimeoutError(
            f"rank {rank}: a device-side wait of a communication kernel gave up (code {comm_code:#x}, "
            f"peer {(comm_code & 0xff) - 1}); the data it was moving is incomplete"
        )
    if kernel_code:
        raise KernelWaitError(
            f"rank {rank}: a bounded barrier wait inside a compute kernel gave up (code {kernel_code:#x}: kernel "
            f"{kernel_code >> 8:#x}, role {kernel_code & 0xff}); its output is incomplete"
        )
