# SPDX-License-Identifier: Apache-2.0
"""Data-type enum accepted by ``model.dtype``.  Parity: arctic_training/config/enums.py:25-64."""

from __future__ import annotations

from enum import Enum

import torch

_ALIASES = {
    torch.float16: ("fp16", "float16", "half", "torch.float16"),
    torch.float32: ("fp32", "float32", "float", "torch.float32"),
    torch.bfloat16: ("bf16", "bfloat16", "bfloat", "torch.bfloat16"),
}


class DType(Enum):
    FP16 = torch.float16
    FP32 = torch.float32
    BF16 = torch.bfloat16

    @classmethod
    def _missing_(cls, value):
        if isinstance(value, DType):
            return value
        if isinstance(value, str):
            key = value.strip().lower()
            for dtype, names in _ALIASES.items():
                if key in names:
                    return cls(dtype)
        raise ValueError(f"{value!r} is not a valid DType")

    def __repr__(self) -> str:
        return f"DType.{self.name}"
