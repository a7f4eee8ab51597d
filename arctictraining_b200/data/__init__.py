# SPDX-License-Identifier: Apache-2.0
from .causal import CausalDataFactory
from .dpo import DPODataFactory
from .factory import DataFactory
from .hf_sources import HFDataSource
from .hf_sources import HFDataSourceCausal
from .hf_sources import HFDataSourceInstruct
from .hf_sources import ProjectGutenbergSFT
from .hf_sources import UltraFeedbackBinarized
from .sft import SFTDataFactory
from .snowflake import SnowflakeDataSource
from .source import DataSource
from .synthetic import SyntheticDataSource
from .synthetic import SyntheticDPOSource
from .synthetic import SyntheticMessagesSource

__all__ = [
    "CausalDataFactory", "DPODataFactory", "DataFactory", "HFDataSource", "HFDataSourceCausal", "HFDataSourceInstruct",
    "ProjectGutenbergSFT", "UltraFeedbackBinarized", "SFTDataFactory", "SnowflakeDataSource", "DataSource",
    "SyntheticDataSource", "SyntheticDPOSource", "SyntheticMessagesSource",
]
