# SPDX-License-Identifier: Apache-2.0
from .losses import info_nce_loss
from .losses import one_size_truncated_mrl_info_nce_loss
from .model import Biencoder
from .model import BiencoderConfig

__all__ = ["info_nce_loss", "one_size_truncated_mrl_info_nce_loss", "Biencoder", "BiencoderConfig"]
