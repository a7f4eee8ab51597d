# SPDX-License-Identifier: Apache-2.0
from .arch import ArchConfig
from .arch import load_arch_config
from .causal_lm import CausalLM
from .causal_lm import CausalLMOutput
from .factory import HFModelFactory
from .factory import LigerModelFactory
from .factory import ModelFactory

__all__ = ["ArchConfig", "load_arch_config", "CausalLM", "CausalLMOutput", "HFModelFactory", "LigerModelFactory", "ModelFactory"]
