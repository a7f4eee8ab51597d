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

    # A member compares equal to its torch dtype and to every alias string, so ``config.dtype == torch.bfloat16`` and
    # ``config.dtype == "bf16"`` both hold; the hash is that of the torch dtype.
    def __eq__(self, other) -> bool:
        if isinstance(other, DType):
            return self is other
        if isinstance(other, str):
            return other.strip().lower() in _ALIASES[self.value]
        return other == self.value

    def __hash__(self) -> int:
        return hash(self.value)

    # Config fields keep the member itself (``config.dtype.value`` is the torch dtype), whatever the model's
    # ``use_enum_values`` setting says; serialisation writes the torch name.
    @classmethod
    def __get_pydantic_core_schema__(cls, source_type, handler):
        from pydantic_core import core_schema

        return core_schema.no_info_after_validator_function(
            cls, core_schema.any_schema(),
            serialization=core_schema.plain_serializer_function_ser_schema(lambda member: str(member.value)),
        )

    @classmethod
    def __get_pydantic_json_schema__(cls, schema, handler):
        return {"type": "string", "title": "Torch Dtype", "examples": ["float32", "bfloat16"]}
