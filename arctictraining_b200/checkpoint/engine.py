# SPDX-License-Identifier: Apache-2.0
"""Checkpoint engine base class.  Parity: arctic_training/checkpoint/engine.py:36-128."""

from __future__ import annotations

from abc import ABC
from abc import abstractmethod
from pathlib import Path
from typing import TYPE_CHECKING
from typing import Any

import torch

from ..callback.mixin import CallbackMixin
from ..callback.mixin import callback_wrapper
from ..config.checkpoint import CheckpointConfig
from ..registry import RegistryMeta
from ..registry import _validate_class_attribute_set
from ..registry import _validate_class_attribute_type
from ..registry import _validate_class_method

if TYPE_CHECKING:
    from ..trainer.trainer import Trainer


class CheckpointEngine(ABC, CallbackMixin, metaclass=RegistryMeta):
    name: str
    """ Name under which the engine is selected in a recipe (``checkpoint[].type``). """

    config: CheckpointConfig
    """ Config class of this engine. """

    @classmethod
    def _validate_subclass(cls) -> None:
        _validate_class_attribute_set(cls, "name")
        _validate_class_attribute_type(cls, "config", CheckpointConfig)
        _validate_class_method(cls, "load", ["self", "model"])
        _validate_class_method(cls, "save", ["self", "model"])

    def __init__(self, trainer: "Trainer", config: CheckpointConfig) -> None:
        self._trainer = trainer
        self.config = config

    @property
    def trainer(self) -> "Trainer":
        return self._trainer

    @property
    def global_rank(self) -> int:
        return self.trainer.global_rank

    @property
    def world_size(self) -> int:
        return self.trainer.world_size

    @property
    def device(self) -> torch.device:
        return self.trainer.device

    @property
    def epoch_finished(self) -> bool:
        return self.trainer.epoch_finished

    @property
    def training_finished(self) -> bool:
        return self.trainer.training_finished

    @property
    def do_checkpoint(self) -> bool:
        """True when the trainer's state sits on one of this engine's save boundaries."""
        cfg = self.config
        if not cfg.enabled:
            return False
        hit = False
        if cfg.save_every_n_steps and self.trainer.model.is_gradient_accumulation_boundary():
            hit = self.trainer.global_step % cfg.save_every_n_steps == 0
        if cfg.save_every_n_epochs:
            hit = hit or (self.epoch_finished and self.trainer.epoch_idx % cfg.save_every_n_epochs == 0)
        if cfg.save_end_of_training:
            hit = hit or self.training_finished
        return hit

    @property
    def checkpoint_dir(self) -> Path:
        d = self.config.output_dir / f"global_step_{self.trainer.global_step}"
        d.mkdir(parents=True, exist_ok=True)
        return d

    @property
    def latest_checkpoint_exists(self) -> bool:
        raise NotImplementedError

    @abstractmethod
    @callback_wrapper("load")
    def load(self, model: Any) -> Any:
        raise NotImplementedError

    @abstractmethod
    @callback_wrapper("save")
    def save(self, model: Any) -> None:
        raise NotImplementedError
