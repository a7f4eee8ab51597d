# SPDX-License-Identifier: Apache-2.0
from .modules import ArcticLSTMSpeculator
from .modules import ArcticLSTMSpeculatorConfig
from .modules import LayerNormParameterized
from .modules import MLPSpeculator
from .modules import MLPSpeculatorConfig
from .modules import Speculator
from .modules import SpeculatorConfig

__all__ = ["ArcticLSTMSpeculator", "ArcticLSTMSpeculatorConfig", "LayerNormParameterized", "MLPSpeculator",
           "MLPSpeculatorConfig", "Speculator", "SpeculatorConfig"]
