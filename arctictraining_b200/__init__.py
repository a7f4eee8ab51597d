# SPDX-License-Identifier: Apache-2.0
"""arctictraining_b200 — a Blackwell-native LLM post-training framework with the public surface of
ArcticTraining (arctic_training/__init__.py:20-57): YAML recipes, registry-driven trainers and factories,
callbacks, Hugging Face and sharded checkpoints."""

from .callback.callback import Callback
from .checkpoint.engine import CheckpointEngine
from .checkpoint.hf import HFCheckpointEngine
from .checkpoint.sharded import DSCheckpointEngine
from .config.checkpoint import CheckpointConfig
from .config.data import DataConfig
from .config.data import DataSourceConfig
from .config.logger import LoggerConfig
from .config.model import ModelConfig
from .config.optimizer import OptimizerConfig
from .config.scheduler import SchedulerConfig
from .config.tokenizer import TokenizerConfig
from .config.trainer import TrainerConfig
from .config.trainer import get_config
from .config.wandb import WandBConfig
from .data.causal import CausalDataFactory
from .data.dpo import DPODataFactory
from .data.factory import DataFactory
from .data.hf_sources import HFDataSource
from .data.hf_sources import HFDataSourceCausal
from .data.hf_sources import HFDataSourceInstruct
from .data.sft import SFTDataFactory
from .data.snowflake import SnowflakeDataSource
from .data.source import DataSource
from .data.synthetic import SyntheticDataSource
from .logging import logger
from .logging import setup_init_logger
from .models.factory import HFModelFactory
from .models.factory import LigerModelFactory
from .models.factory import ModelFactory
from .optimizer.adam import FusedAdamOptimizerFactory
from .optimizer.factory import OptimizerFactory
from .registry import register
from .scheduler.factory import HFSchedulerFactory
from .scheduler.factory import SchedulerFactory
from .tokenizer.factory import HFTokenizerFactory
from .tokenizer.factory import TokenizerFactory
from .trainer.sft import CausalTrainer
from .trainer.sft import SFTTrainer
from .trainer.trainer import Trainer
from .trainer.dpo import DPOTrainer
from .trainer.dpo import DPOTrainerConfig

__version__ = "0.1.0"
