# SPDX-License-Identifier: Apache-2.0
"""``wandb:`` section.  Parity: arctic_training/config/wandb.py:21-32."""

from __future__ import annotations

from typing import Optional

from .base import BaseConfig


class WandBConfig(BaseConfig):
    enable: bool = False
    """ Whether to log to Weights and Biases (rank 0 only). """

    entity: Optional[str] = None
    """ Entity name. """

    project: Optional[str] = "arctic-training"
    """ Project name. """

    name: Optional[str] = None
    """ Run name. """
