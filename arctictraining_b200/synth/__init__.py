# SPDX-License-Identifier: Apache-2.0
from .base import BatchProcessor
from .base import InMemoryBatchProcessor
from .callers import CortexSynth
from .callers import MultiReplicaVllmSynth
from .callers import VllmSynth
from .openai_callers import AzureOpenAISynth
from .openai_callers import OpenAIBatchProcessor
from .openai_callers import OpenAISynth

__all__ = ["BatchProcessor", "InMemoryBatchProcessor", "CortexSynth", "MultiReplicaVllmSynth", "VllmSynth",
           "AzureOpenAISynth", "OpenAIBatchProcessor", "OpenAISynth"]
