# SPDX-License-Identifier: Apache-2.0
from .base import BaseConfig
from .checkpoint import CheckpointConfig
from .data import DataConfig
from .data import DataSourceConfig
from .enums import DType
from .logger import LoggerConfig
from .model import ModelConfig
from .optimizer import OptimizerConfig
from .scheduler import SchedulerConfig
from .tokenizer import TokenizerConfig
from .trainer import TrainerConfig
from .trainer import get_config
from .utils import HumanFloat
from .utils import HumanInt
from .wandb import WandBConfig

__all__ = [
    "BaseConfig", "CheckpointConfig", "DataConfig", "DataSourceConfig", "DType", "LoggerConfig", "ModelConfig",
    "OptimizerConfig", "SchedulerConfig", "TokenizerConfig", "TrainerConfig", "get_config", "HumanFloat",
    "HumanInt", "WandBConfig",
]
