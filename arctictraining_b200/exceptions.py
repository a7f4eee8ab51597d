# SPDX-License-Identifier: Apache-2.0
"""Error types raised by the registry and the communication layer."""


class RegistryError(Exception):
    """A lookup in the class registry failed (unknown base type or unknown name)."""


class RegistryValidationError(Exception):
    """A class failed validation at declaration time (missing name, wrong signature, duplicate)."""


class CommTimeoutError(RuntimeError):
    """A bounded device-side wait on a peer flag ran out; the context stays usable."""


class EngineConfigError(ValueError):
    """The engine section of a recipe asks for a combination that is not supported."""


class KernelWaitError(RuntimeError):
    """A bounded barrier wait inside a compute kernel (GEMM, attention) ran out; its output is incomplete."""


class CheckpointError(RuntimeError):
    """A checkpoint cannot be used: a file is missing, truncated or unreadable, or it does not fit this run's layout."""
