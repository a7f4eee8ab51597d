# SPDX-License-Identifier: Apache-2.0
"""Moves (nested) batches to a device.  Parity: arctic_training/trainer/utils.py:21-28."""

from __future__ import annotations

from typing import Any

import torch


def to_device(batch: Any, device: torch.device) -> Any:
    if torch.is_tensor(batch):
        return batch.to(device, non_blocking=True)
    if isinstance(batch, dict):
        return {k: to_device(v, device) for k, v in batch.items()}
    if isinstance(batch, (list, tuple)):
        return type(batch)(to_device(v, device) for v in batch)
    return batch
