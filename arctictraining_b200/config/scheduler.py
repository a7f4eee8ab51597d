# SPDX-License-Identifier: Apache-2.0
"""``scheduler:`` section.  Parity: arctic_training/config/scheduler.py:30-46."""

from __future__ import annotations

from typing import TYPE_CHECKING
from typing import Optional
from typing import Type

from pydantic import Field
from pydantic import field_validator

from ..registry import get_registered_scheduler_factory
from .base import BaseConfig

if TYPE_CHECKING:
    from ..scheduler.factory import SchedulerFactory


class SchedulerConfig(BaseConfig):
    type: str = ""
    """ Scheduler factory type. Defaults to the first ``scheduler_factory`` hint of the trainer. """

    learning_rate: Optional[float] = Field(default=None, alias="lr")
    """ Deprecated: the learning rate lives in ``optimizer.learning_rate``. """

    @field_validator("learning_rate", mode="after")
    @classmethod
    def _moved(cls, value: Optional[float]) -> Optional[float]:
        if value is not None:
            raise ValueError("scheduler.learning_rate is deprecated. Use optimizer.learning_rate instead.")
        return value

    @property
    def factory(self) -> Type["SchedulerFactory"]:
        return get_registered_scheduler_factory(name=self.type)
