# SPDX-License-Identifier: Apache-2.0
"""Host offload for code that checkpoints activations through ``torch.utils.checkpoint`` itself (library models, user
modules): the tensors a checkpointed region keeps for its backward pass - its inputs, i.e. the hidden state that enters
a layer - wait in pinned host memory instead of on the device.

Models that run under this package's engine do not need this - own architectures and transformers models alike: the
engine checkpoints their decoder layers itself and offloads the layer inputs through the same
:class:`~arctictraining_b200.engine.activation.ActivationStore` (``activation_checkpoint_cpu_offload: true``).  This
module is for code that calls ``torch.utils.checkpoint`` on its own, outside those layers.

How: ``torch.utils.checkpoint.checkpoint`` is wrapped so that the call runs in its re-entrant form under a pair of
saved-tensor hooks.  The re-entrant form saves exactly its tensor arguments; the pack hook hands every large floating
device tensor to the store (asynchronous copy on a side stream into a pooled pinned buffer), the unpack hook brings it
back and starts the prefetch of the tensor saved before it, so the copy for layer ``i-1`` overlaps the recompute of
layer ``i``.  The reference replaces the checkpoint autograd function with a copy that moves argument 0 with a
synchronous ``.cpu()`` / ``.to(device)`` pair (arctic_training/monkey_patches.py:37-169).
"""

from __future__ import annotations

import functools
from typing import Any
from typing import Callable
from typing import Dict
from typing import Optional

import torch
import torch.utils.checkpoint as _ckpt

from .engine.activation import ActivationStore
from .engine.activation import _Handle

_original_checkpoint: Optional[Callable[..., Any]] = None
_stores: Dict[torch.device, ActivationStore] = {}
stats = {"packed": 0, "restored": 0}


def noop_context_fn():
    """The default ``context_fn`` of ``torch.utils.checkpoint.checkpoint``: two null contexts."""
    import contextlib

    return contextlib.nullcontext(), contextlib.nullcontext()


def _store_for(device: torch.device) -> ActivationStore:
    store = _stores.get(device)
    if store is None:
        store = _stores[device] = ActivationStore(device, offload=True)
    return store


class offload_checkpoint_inputs(torch.autograd.graph.saved_tensors_hooks):  # noqa: N801 - used as a context manager
    """Saved-tensor hooks that park large floating tensors in pinned host memory until backward needs them."""

    def __init__(self, min_bytes: int = 1 << 20) -> None:
        def pack(x: torch.Tensor):
            if not x.is_floating_point() or x.numel() * x.element_size() < min_bytes:
                return x
            stats["packed"] += 1
            return _store_for(x.device).save(x)

        def unpack(saved):
            if isinstance(saved, _Handle):
                stats["restored"] += 1
                return saved.restore()
            return saved

        super().__init__(pack, unpack)


_torch_checkpoint = _ckpt.checkpoint
DEFAULT_MIN_BYTES = 1 << 20


def checkpoint_with_host_offload(function, *args, min_bytes: Optional[int] = None, **kwargs):
    """``torch.utils.checkpoint.checkpoint`` whose saved inputs wait in host memory.  Usable directly as the
    ``gradient_checkpointing_func`` of a Hugging Face model."""
    # only the re-entrant form saves its inputs through the autograd machinery, where the hooks can see them
    for unsupported in ("use_reentrant", "context_fn", "determinism_check", "debug"):
        kwargs.pop(unsupported, None)
    with offload_checkpoint_inputs(DEFAULT_MIN_BYTES if min_bytes is None else min_bytes):
        return _torch_checkpoint(function, *args, use_reentrant=True, **kwargs)


def enable_host_offload_on_hf_model(model: torch.nn.Module) -> bool:
    """Point a Hugging Face model's gradient checkpointing at :func:`checkpoint_with_host_offload`.  Those models bind
    the checkpoint function when checkpointing is enabled, so patching the torch module afterwards would not reach
    them.  Returns False when the model has no such switch."""
    setter = getattr(model, "_set_gradient_checkpointing", None)
    if setter is None:
        return False
    setter(enable=True, gradient_checkpointing_func=checkpoint_with_host_offload)
    return True


def monkey_patch_checkpoint_function_with_cpu_offload(min_bytes: int = DEFAULT_MIN_BYTES) -> None:
    """Make every later ``torch.utils.checkpoint.checkpoint(...)`` call keep its inputs in host memory.  Idempotent;
    :func:`undo_checkpoint_patch` restores the original function.  Code that imported the function by name before the
    patch keeps the original: call this first, or use :func:`enable_host_offload_on_hf_model`."""
    global _original_checkpoint
    if _original_checkpoint is not None:
        return
    _original_checkpoint = _ckpt.checkpoint
    patched = functools.wraps(_torch_checkpoint)(functools.partial(checkpoint_with_host_offload, min_bytes=min_bytes))
    _ckpt.checkpoint = patched
    torch.utils.checkpoint.checkpoint = patched


def undo_checkpoint_patch() -> None:
    global _original_checkpoint
    if _original_checkpoint is not None:
        _ckpt.checkpoint = _original_checkpoint
        torch.utils.checkpoint.checkpoint = _original_checkpoint
        _original_checkpoint = None
