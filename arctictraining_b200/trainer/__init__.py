# SPDX-License-Identifier: Apache-2.0
from .sft import CausalTrainer
from .sft import SFTTrainer
from .trainer import Trainer

__all__ = ["CausalTrainer", "SFTTrainer", "Trainer"]
