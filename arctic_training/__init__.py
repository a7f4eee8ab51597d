# SPDX-License-Identifier: Apache-2.0
"""Import-name compatibility: ``import arctic_training`` resolves to :mod:`arctictraining_b200`, so user
``train.py`` files and recipes written against the reference's package name keep working."""

import importlib
import sys

import arctictraining_b200 as _impl
from arctictraining_b200 import *  # noqa: F401,F403

_ALIASES = {
    "registry": "registry", "config": "config", "callback": "callback", "logging": "logging", "metrics": "metrics",
    "trainer": "trainer", "data": "data", "tokenizer": "tokenizer", "optimizer": "optimizer", "scheduler": "scheduler",
    "checkpoint": "checkpoint", "model": "models", "debug": "debug", "exceptions": "exceptions", "utils": "utils.misc",
    "synth": "synth", "launcher": "launcher",
}
for _old, _new in _ALIASES.items():
    try:
        sys.modules[f"arctic_training.{_old}"] = importlib.import_module(f"arctictraining_b200.{_new}")
    except ImportError:
        pass
for _name in dir(_impl):
    if not _name.startswith("__"):
        globals().setdefault(_name, getattr(_impl, _name))
