# SPDX-License-Identifier: Apache-2.0
"""MLP speculator project: importing this file registers the ``spec-decode`` trainer, model factory and checkpoint
engine (implementation: ``arctictraining_b200/speculator``)."""

from arctictraining_b200.speculator.trainer import MLPSpeculatorCheckpointEngine  # noqa: F401
from arctictraining_b200.speculator.trainer import MLPSpeculatorModelFactory  # noqa: F401
from arctictraining_b200.speculator.trainer import MLPSpeculatorTrainer  # noqa: F401
