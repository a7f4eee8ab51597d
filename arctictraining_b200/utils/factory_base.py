# SPDX-License-Identifier: Apache-2.0
"""Accessors shared by all factory base classes (they all hold a reference to the trainer)."""

from __future__ import annotations

from typing import TYPE_CHECKING

if TYPE_CHECKING:
    from ..trainer.trainer import Trainer


class TrainerBound:
    _trainer: "Trainer"

    @property
    def trainer(self) -> "Trainer":
        return self._trainer

    @property
    def device(self):
        return self._trainer.device

    @property
    def world_size(self) -> int:
        return self._trainer.world_size

    @property
    def global_rank(self) -> int:
        return self._trainer.global_rank

    @property
    def local_rank(self) -> int:
        return self._trainer.config.local_rank
