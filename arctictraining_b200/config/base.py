# SPDX-License-Identifier: Apache-2.0
"""Base class of every config object.  Parity: arctic_training/config/base.py:26-42."""

from __future__ import annotations

from pydantic import BaseModel
from pydantic import ConfigDict
from pydantic import Field

from .utils import get_global_rank
from .utils import get_local_rank
from .utils import get_world_size


class BaseConfig(BaseModel):
    model_config = ConfigDict(
        extra="forbid",
        use_enum_values=True,
        validate_assignment=True,
        validate_default=True,
        use_attribute_docstrings=True,
        populate_by_name=True,
        arbitrary_types_allowed=True,
    )

    local_rank: int = Field(default_factory=get_local_rank, exclude=True)
    global_rank: int = Field(default_factory=get_global_rank, exclude=True)
    world_size: int = Field(default_factory=get_world_size, exclude=True)
