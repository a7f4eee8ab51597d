# SPDX-License-Identifier: Apache-2.0
"""Small helpers of the data-generation clients.  Parity: arctic_training/synth/utils.py:17-40."""

from __future__ import annotations

from typing import Any


def import_error(**kwargs: Any) -> None:
    """Stands in for a class of an optional package that is not installed: using it says what to install."""
    raise ImportError("Please install the vllm package to use this class.")


def pass_function(**kwargs: Any) -> None:
    return None


def recursive_to_dict(obj: Any) -> Any:
    """Plain dicts / lists / tuples / scalars out of nested objects (SDK response objects become JSON-serialisable):
    anything with a ``__dict__`` is replaced by the conversion of its attributes."""
    if isinstance(obj, dict):
        return {k: recursive_to_dict(v) for k, v in obj.items()}
    if isinstance(obj, list):
        return [recursive_to_dict(v) for v in obj]
    if isinstance(obj, tuple):
        return tuple(recursive_to_dict(v) for v in obj)
    if hasattr(obj, "__dict__"):
        return recursive_to_dict(vars(obj))
    return obj
