# SPDX-License-Identifier: Apache-2.0
from .config import EngineConfig
from .engine import TrainingEngine
from .engine import initialize

__all__ = ["EngineConfig", "TrainingEngine", "initialize"]
