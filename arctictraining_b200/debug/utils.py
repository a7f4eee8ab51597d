# SPDX-License-Identifier: Apache-2.0
"""Memory and rank-aware printing helpers.  Parity: arctic_training/debug/utils.py:50-287."""

from __future__ import annotations

import fcntl
import gc
import os
from typing import Any
from typing import List
from typing import Optional

import torch
import torch.distributed as dist

DISABLE_SEE_MEM_USAGE = True
_nvml_handle = None


def _rank() -> int:
    return dist.get_rank() if dist.is_initialized() else int(os.getenv("RANK", 0))


def printflock(*args: Any, **kwargs: Any) -> None:
    """``print`` under an exclusive file lock so lines of different ranks do not interleave."""
    with open(__file__, "r") as fh:
        fcntl.flock(fh, fcntl.LOCK_EX)
        try:
            print(*args, **kwargs)
        finally:
            fcntl.flock(fh, fcntl.LOCK_UN)


def print_rank(*msg: Any, skip: bool = True, ranks: Optional[List[int]] = None, force: bool = False) -> None:
    if skip and not force:
        return
    if ranks is None or _rank() in ranks:
        printflock(f"[{_rank()}]", *msg)


def pr0(*msg: Any, skip: bool = True, force: bool = False) -> None:
    print_rank(*msg, skip=skip, ranks=[0], force=force)


def _nvml_used_gb() -> Optional[float]:
    global _nvml_handle
    if not torch.cuda.is_available():
        return None
    try:
        import pynvml

        if _nvml_handle is None:
            pynvml.nvmlInit()
            _nvml_handle = pynvml.nvmlDeviceGetHandleByIndex(torch.cuda.current_device())
        return pynvml.nvmlDeviceGetMemoryInfo(_nvml_handle).used / 2**30
    except Exception:
        return None


def get_mem_metrics() -> str:
    """``MA/Max_MA`` (torch allocator), ``NV`` (device memory in use as NVML reports it) and CPU RSS, in GB."""
    parts = []
    if torch.cuda.is_available():
        parts.append(f"MA {torch.cuda.memory_allocated() / 2**30:.2f} GB")
        parts.append(f"Max_MA {torch.cuda.max_memory_allocated() / 2**30:.2f} GB")
        nv = _nvml_used_gb()
        if nv is not None:
            parts.append(f"NV {nv:.2f} GB")
    try:
        import psutil

        parts.append(f"CPU RSS {psutil.Process().memory_info().rss / 2**30:.2f} GB")
        vm = psutil.virtual_memory()
        parts.append(f"node RAM {vm.used / 2**30:.1f}/{vm.total / 2**30:.1f} GB")
    except Exception:
        pass
    return " | ".join(parts)


def see_memory_usage(message: str, force: bool = False, ranks: Optional[List[int]] = None) -> None:
    if DISABLE_SEE_MEM_USAGE and not force:
        return
    if ranks is not None and _rank() not in ranks:
        return
    gc.collect()
    printflock(f"[{_rank()}] {message} | {get_mem_metrics()}")
    if torch.cuda.is_available():
        torch.cuda.reset_peak_memory_stats()


def tensor_has_nan(t: torch.Tensor) -> bool:
    return bool(torch.isnan(t).any() or torch.isinf(t).any())


def debug_gathered_tensor(tensor: torch.Tensor, group=None, name: str = "tensor", dim: int = 0) -> torch.Tensor:
    """All-gather a tensor over ``group`` and print its summary on rank 0 (debugging aid)."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        full = tensor
    else:
        parts = [torch.empty_like(tensor) for _ in range(dist.get_world_size(group))]
        dist.all_gather(parts, tensor.contiguous(), group=group)
        full = torch.cat(parts, dim=dim)
    if _rank() == 0:
        f = full.float()
        printflock(f"{name}: shape={tuple(full.shape)} norm={f.norm():.6f} mean={f.mean():.6f} absmax={f.abs().max():.6f}")
    return full
