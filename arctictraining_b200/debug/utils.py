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


def print_rank0(*msg: Any, skip: bool = True, force: bool = False) -> None:
    print_rank(*msg, skip=skip, ranks=[0], force=force)


pr0 = print_rank0
pr = print_rank


def get_device_id(current_device: Optional[int] = None):
    """Physical index (or UUID string) of the GPU this process computes on, as management tools number it:
    ``CUDA_VISIBLE_DEVICES`` re-numbers devices inside the process, NVML does not.  ``None`` when no device is visible."""
    visible = os.getenv("CUDA_VISIBLE_DEVICES")
    if current_device is None:
        current_device = torch.cuda.current_device() if torch.cuda.is_available() else int(os.getenv("LOCAL_RANK", 0))
    if visible is None:
        return current_device
    entries = [e.strip() for e in visible.split(",") if e.strip()]
    if not entries:
        return None
    entry = entries[current_device] if current_device < len(entries) else entries[0]
    return int(entry) if entry.lstrip("-").isdigit() else entry


def get_nvml_mem() -> int:
    """Bytes in use on this process' GPU as NVML reports them (all processes, allocator caches included); 0 when NVML
    is not available or does not support the query on this machine."""
    global _nvml_handle
    try:
        import pynvml

        if _nvml_handle is None:
            device = get_device_id()
            if device is None:
                return 0
            pynvml.nvmlInit()
            by_uuid = isinstance(device, str)
            _nvml_handle = (pynvml.nvmlDeviceGetHandleByUUID(device) if by_uuid
                            else pynvml.nvmlDeviceGetHandleByIndex(device))
        return int(pynvml.nvmlDeviceGetMemoryInfo(_nvml_handle).used)
    except Exception:
        return 0


def _nvml_used_gb() -> Optional[float]:
    if not torch.cuda.is_available():
        return None
    used = get_nvml_mem()
    return used / 2**30 if used else None


def gc_empty_accelerator_cache() -> None:
    """Collect garbage and return the allocator's cached blocks to the device: for reading real memory use while
    debugging (expensive, not for the training loop)."""
    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.empty_cache()


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
