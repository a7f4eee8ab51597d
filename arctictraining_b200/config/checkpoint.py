# SPDX-License-Identifier: Apache-2.0
"""One entry of the ``checkpoint:`` list.  Parity: arctic_training/config/checkpoint.py:31-60."""

from __future__ import annotations

from pathlib import Path
from typing import TYPE_CHECKING
from typing import Type

from pydantic import Field
from pydantic import field_validator

from ..registry import get_registered_checkpoint_engine
from .base import BaseConfig
from .utils import HumanInt

if TYPE_CHECKING:
    from ..checkpoint.engine import CheckpointEngine


class CheckpointConfig(BaseConfig):
    type: str = ""
    """ Checkpoint engine type (``deepspeed``: resumable sharded layout, ``huggingface``: export layout). """

    output_dir: Path
    """ Checkpoint output directory; created when missing. """

    enabled: bool = True
    """ Enable this checkpoint engine. """

    auto_resume: bool = False
    """ Resume from the newest checkpoint found in ``output_dir``. """

    save_every_n_steps: HumanInt = Field(default=0, ge=0)
    """ Save every this many optimizer steps (0: never). """

    save_every_n_epochs: HumanInt = Field(default=0, ge=0)
    """ Save every this many epochs (0: never). """

    save_end_of_training: bool = False
    """ Save once when training finishes. """

    @property
    def engine(self) -> Type["CheckpointEngine"]:
        return get_registered_checkpoint_engine(name=self.type)

    @field_validator("output_dir", mode="after")
    @classmethod
    def _absolute(cls, v: Path) -> Path:
        return v.resolve()
