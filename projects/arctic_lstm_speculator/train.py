# SPDX-License-Identifier: Apache-2.0
"""Arctic LSTM speculator project: importing this file registers the ``arctic-lstm-speculator`` trainer, model factory
and checkpoint engine (implementation: ``arctictraining_b200/speculator``)."""

from arctictraining_b200.speculator.trainer import ArcticLSTMSpeculatorCheckpointEngine  # noqa: F401
from arctictraining_b200.speculator.trainer import ArcticLSTMSpeculatorModelFactory  # noqa: F401
from arctictraining_b200.speculator.trainer import ArcticLSTMSpeculatorTrainer  # noqa: F401
