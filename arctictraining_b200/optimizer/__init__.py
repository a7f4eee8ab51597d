# SPDX-License-Identifier: Apache-2.0
from .adam import CPUAdamMoEOptimizerFactory
from .adam import CPUAdamOptimizerFactory
from .adam import CPUAdamW
from .adam import FusedAdamMoEOptimizerFactory
from .adam import FusedAdamOptimizerFactory
from .adam import FusedAdamW
from .factory import OptimizerFactory

__all__ = [
    "CPUAdamMoEOptimizerFactory", "CPUAdamOptimizerFactory", "CPUAdamW", "FusedAdamMoEOptimizerFactory",
    "FusedAdamOptimizerFactory", "FusedAdamW", "OptimizerFactory",
]
