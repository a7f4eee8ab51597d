# SPDX-License-Identifier: Apache-2.0
from .base import BatchProcessor
from .base import InMemoryBatchProcessor
from .callers import CortexSynth
from .callers import MultiReplicaVllmSynth
from .callers import VllmSynth
from .openai_callers import AzureOpenAISynth
from .openai_callers import OpenAIBatchProcessor
from .openai_callers import OpenAISynth


def main(argv=None):
    """The ``arctic_synth`` command (imported lazily: the CLI pulls in optional clients)."""
    from .cli import main as _main

    return _main(argv)

__all__ = ["BatchProcessor", "InMemoryBatchProcessor", "CortexSynth", "MultiReplicaVllmSynth", "VllmSynth",
           "AzureOpenAISynth", "OpenAIBatchProcessor", "OpenAISynth", "main"]
