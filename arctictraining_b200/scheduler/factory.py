# SPDX-License-Identifier: Apache-2.0
"""Scheduler factories.  Parity: arctic_training/scheduler/factory.py:34-94, hf_factory.py:26-46,
wsd_factory.py:25-46 (the WSD factory keeps the reference's registered name ``wds``)."""

from __future__ import annotations

from abc import ABC
from abc import abstractmethod
from typing import TYPE_CHECKING
from typing import Any
from typing import Dict
from typing import Optional

from pydantic import Field

from ..callback.mixin import CallbackMixin
from ..callback.mixin import callback_wrapper
from ..config.scheduler import SchedulerConfig
from ..config.utils import HumanFloat
from ..registry import RegistryMeta
from ..registry import _validate_class_attribute_set
from ..registry import _validate_class_attribute_type
from ..registry import _validate_class_method
from ..utils.factory_base import TrainerBound
from .schedules import get_scheduler
from .schedules import get_wsd_schedule

if TYPE_CHECKING:
    from ..trainer.trainer import Trainer


class SchedulerFactory(ABC, CallbackMixin, TrainerBound, metaclass=RegistryMeta):
    name: str
    """ Name under which the factory is selected in a recipe (``scheduler.type``). """

    config: SchedulerConfig
    """ Config class of this factory. """

    @classmethod
    def _validate_subclass(cls) -> None:
        _validate_class_attribute_set(cls, "name")
        _validate_class_attribute_type(cls, "config", SchedulerConfig)
        _validate_class_method(cls, "create_scheduler", ["self", "optimizer"])

    def __init__(self, trainer: "Trainer", scheduler_config: Optional[SchedulerConfig] = None) -> None:
        self._trainer = trainer
        self.config = scheduler_config if scheduler_config is not None else trainer.config.scheduler

    def __call__(self) -> Any:
        return self.create_scheduler(optimizer=self.optimizer)

    @property
    def optimizer(self) -> Any:
        return self.trainer.optimizer

    @abstractmethod
    @callback_wrapper("create-scheduler")
    def create_scheduler(self, optimizer: Any) -> Any:
        raise NotImplementedError


class HFSchedulerConfig(SchedulerConfig):
    name: str = "linear"
    """ Schedule family: linear, cosine, constant, constant_with_warmup, polynomial, inverse_sqrt ... """

    warmup_ratio: HumanFloat = Field(default=0.1, ge=0.0, le=1.0)
    """ Fraction of the training horizon used for linear warm-up. """

    scheduler_specific_kwargs: Dict[str, Any] = Field(default_factory=dict)
    """ Extra keyword arguments of the schedule. """


class HFSchedulerFactory(SchedulerFactory):
    name = "huggingface"
    config: HFSchedulerConfig

    def create_scheduler(self, optimizer: Any) -> Any:
        # under sequence parallelism one dataloader step is SP micro-steps, hence the factor
        sp = self.trainer.config.sequence_parallel_size
        horizon = self.trainer.training_horizon
        return get_scheduler(
            self.config.name, optimizer,
            num_warmup_steps=int(self.config.warmup_ratio * horizon) * sp,
            num_training_steps=horizon * sp,
            scheduler_specific_kwargs=self.config.scheduler_specific_kwargs,
        )


class WSDSchedulerConfig(SchedulerConfig):
    name: str = "wsd"
    num_warmup_steps: int
    num_decay_steps: int
    min_lr_ratio: float = 0.0


class WSDSchedulerFactory(SchedulerFactory):
    name = "wds"
    config: WSDSchedulerConfig

    def create_scheduler(self, optimizer: Any) -> Any:
        stable = self.trainer.training_horizon - self.config.num_warmup_steps - self.config.num_decay_steps
        return get_wsd_schedule(optimizer, self.config.num_warmup_steps, stable, self.config.num_decay_steps,
                                self.config.min_lr_ratio)
