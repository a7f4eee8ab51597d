# SPDX-License-Identifier: Apache-2.0
from .convert import convert_to_arctic_moe
from .convert import detect_if_moe_model
from .layer import ArcticMoE
from .layer import MoEConfig
from .layer import build_moe_block

__all__ = ["ArcticMoE", "MoEConfig", "build_moe_block", "convert_to_arctic_moe", "detect_if_moe_model"]
