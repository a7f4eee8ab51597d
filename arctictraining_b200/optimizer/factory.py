# SPDX-License-Identifier: Apache-2.0
"""Optimizer factory base class.  Parity: arctic_training/optimizer/factory.py:34-95."""

from __future__ import annotations

from abc import ABC
from abc import abstractmethod
from typing import TYPE_CHECKING
from typing import Any
from typing import Dict
from typing import List
from typing import Optional

import torch

from ..callback.mixin import CallbackMixin
from ..callback.mixin import callback_wrapper
from ..config.optimizer import OptimizerConfig
from ..registry import RegistryMeta
from ..registry import _validate_class_attribute_set
from ..registry import _validate_class_attribute_type
from ..registry import _validate_class_method
from ..utils.factory_base import TrainerBound

if TYPE_CHECKING:
    from ..trainer.trainer import Trainer

_NO_DECAY_MARKERS = ("bias", "norm.weight", "layernorm.weight", "ln_f.weight", "_norm.weight")


class OptimizerFactory(ABC, CallbackMixin, TrainerBound, metaclass=RegistryMeta):
    name: str
    """ Name under which the factory is selected in a recipe (``optimizer.type``). """

    config: OptimizerConfig
    """ Config class of this factory. """

    @classmethod
    def _validate_subclass(cls) -> None:
        _validate_class_attribute_set(cls, "name")
        _validate_class_attribute_type(cls, "config", OptimizerConfig)
        _validate_class_method(cls, "create_optimizer", ["self", "model", "optimizer_config"])

    def __init__(self, trainer: "Trainer", optimizer_config: Optional[OptimizerConfig] = None) -> None:
        self._trainer = trainer
        self.config = optimizer_config if optimizer_config is not None else trainer.config.optimizer

    def __call__(self) -> Any:
        return self.create_optimizer(self.trainer.model, self.config)

    @property
    def model(self) -> Any:
        return self.trainer.model

    @staticmethod
    def get_optimizer_grouped_params(model: torch.nn.Module, weight_decay: float) -> List[Dict[str, Any]]:
        """Two groups of trainable parameters: with weight decay, and without (biases, norm weights)."""
        decay, no_decay = [], []
        for n, p in model.named_parameters():
            if not p.requires_grad:
                continue
            low = n.lower()
            (no_decay if any(m in low for m in _NO_DECAY_MARKERS) or p.dim() <= 1 and "norm" in low else decay).append(p)
        return [
            {"params": decay, "weight_decay": weight_decay},
            {"params": no_decay, "weight_decay": 0.0},
        ]

    @abstractmethod
    @callback_wrapper("create-optimizer")
    def create_optimizer(self, model: Any, optimizer_config: "OptimizerConfig") -> Any:
        raise NotImplementedError
