# SPDX-License-Identifier: Apache-2.0
from .engine import CheckpointEngine
from .hf import HFCheckpointEngine
from .sharded import DSCheckpointEngine

__all__ = ["CheckpointEngine", "HFCheckpointEngine", "DSCheckpointEngine"]
