# SPDX-License-Identifier: Apache-2.0
from .factory import HFSchedulerConfig
from .factory import HFSchedulerFactory
from .factory import SchedulerFactory
from .factory import WSDSchedulerConfig
from .factory import WSDSchedulerFactory

__all__ = ["HFSchedulerConfig", "HFSchedulerFactory", "SchedulerFactory", "WSDSchedulerConfig", "WSDSchedulerFactory"]
