# SPDX-License-Identifier: Apache-2.0
"""Process-group bootstrap and small helpers used all over the framework.

One process drives one GPU.  ``torch.distributed`` (NCCL on GPUs, Gloo on CPU-only hosts) is the
control plane and the baseline data plane; the fused kernels of ``arctictraining_b200.comm.symm`` use
peer memory directly.  Parity: the reference initialises its process group while the recipe is being
validated (arctic_training/config/trainer.py:201-208); ``init_distributed`` is idempotent and safe to
call from there.
"""

from __future__ import annotations

import datetime
import os
from typing import Any
from typing import List
from typing import Optional

import torch
import torch.distributed as dist


def cuda_available() -> bool:
    return torch.cuda.is_available()


def current_device() -> torch.device:
    if cuda_available():
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def init_distributed(local_rank: Optional[int] = None, timeout_s: Optional[float] = None) -> None:
    """Create the default process group from the launcher's environment (idempotent)."""
    if local_rank is None:
        local_rank = int(os.getenv("LOCAL_RANK", 0))
    if cuda_available():
        torch.cuda.set_device(local_rank % max(torch.cuda.device_count(), 1))
    if dist.is_initialized():
        return
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("LOCAL_RANK", str(local_rank))
    backend = "nccl" if cuda_available() else "gloo"
    kwargs: dict = {}
    if timeout_s is None and os.getenv("ATB200_PG_TIMEOUT_S"):
        timeout_s = float(os.environ["ATB200_PG_TIMEOUT_S"])
    if timeout_s is not None:
        kwargs["timeout"] = datetime.timedelta(seconds=timeout_s)
    if backend == "nccl":
        kwargs["device_id"] = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group(backend=backend, **kwargs)


def get_rank(group: Optional[dist.ProcessGroup] = None) -> int:
    return dist.get_rank(group) if dist.is_initialized() else 0


def get_world_size(group: Optional[dist.ProcessGroup] = None) -> int:
    return dist.get_world_size(group) if dist.is_initialized() else 1


def barrier(group: Optional[dist.ProcessGroup] = None) -> None:
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        if cuda_available():
            dist.barrier(group=group, device_ids=[torch.cuda.current_device()])
        else:
            dist.barrier(group=group)


def all_gather_object(obj: Any, group: Optional[dist.ProcessGroup] = None) -> List[Any]:
    if get_world_size(group) == 1:
        return [obj]
    out: List[Any] = [None] * get_world_size(group)
    dist.all_gather_object(out, obj, group=group)
    return out


def destroy() -> None:
    if dist.is_initialized():
        dist.destroy_process_group()
