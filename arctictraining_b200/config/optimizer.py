# SPDX-License-Identifier: Apache-2.0
"""``optimizer:`` section.  Parity: arctic_training/config/optimizer.py:30-45."""

from __future__ import annotations

from typing import TYPE_CHECKING
from typing import Tuple
from typing import Type

from pydantic import Field

from ..registry import get_registered_optimizer_factory
from .base import BaseConfig
from .utils import HumanFloat

if TYPE_CHECKING:
    from ..optimizer.factory import OptimizerFactory


class OptimizerConfig(BaseConfig):
    type: str = ""
    """ Optimizer factory type. Defaults to the first ``optimizer_factory`` hint of the trainer. """

    weight_decay: HumanFloat = Field(default=0.1, ge=0.0)
    """ Decoupled weight-decay coefficient (not applied to biases and norm weights). """

    betas: Tuple[float, float] = (0.9, 0.999)
    """ Adam running-average coefficients. """

    eps: HumanFloat = Field(default=1e-8, gt=0.0)
    """ Adam epsilon. """

    learning_rate: HumanFloat = Field(default=5e-4, ge=0.0, alias="lr")
    """ The initial learning rate. """

    @property
    def factory(self) -> Type["OptimizerFactory"]:
        return get_registered_optimizer_factory(name=self.type)
