# SPDX-License-Identifier: Apache-2.0
"""Import-name compatibility: ``import arctic_training`` resolves to :mod:`arctictraining_b200`, so user ``train.py``
files, recipes and tests written against the reference's package name keep working — including the reference's module
paths (``arctic_training.trainer.sft_trainer``, ``arctic_training.checkpoint.ds_engine``,
``arctic_training.model.hf_factory`` ...).  An import hook hands out the module of this package that holds the same
classes; nothing is executed twice, so classes register once."""

import importlib
import importlib.abc
import importlib.machinery
import os
import sys

import arctictraining_b200 as _impl
from arctictraining_b200 import *  # noqa: F401,F403

_PREFIX = "arctic_training."
# reference module path (below ``arctic_training.``) -> module of this package (below ``arctictraining_b200.``)
_MODULES = {
    "trainer.sft_trainer": "trainer.sft", "trainer.causal_trainer": "trainer.sft", "trainer.dpo_trainer": "trainer.dpo",
    "checkpoint.ds_engine": "checkpoint.sharded", "checkpoint.hf_engine": "checkpoint.hf",
    "data.sft_factory": "data.sft", "data.causal_factory": "data.causal", "data.dpo_factory": "data.dpo",
    "data.hf_source": "data.hf_sources", "data.hf_instruct_source": "data.hf_sources", "data.hf_causal_source": "data.hf_sources",
    "data.snowflake_source": "data.snowflake",
    "model": "models", "model.factory": "models.factory", "model.hf_factory": "models.factory",
    "model.liger_factory": "models.factory", "model.moe": "moe", "model.moe.moe": "moe.layer", "model.moe.utils": "moe.convert",
    "model.moe.timers": "moe.timers", "model.tiled_compute": "ops.tiled",
    "optimizer.adam_factory": "optimizer.adam",
    "scheduler.hf_factory": "scheduler.factory", "scheduler.wsd_factory": "scheduler.factory",
    "tokenizer.hf_factory": "tokenizer.factory",
    "model.moe.moe_gemm": "moe.grouped",
    "synth.base_caller": "synth.base", "synth.vllm_callers": "synth.callers", "synth.vllm_utils": "synth.callers",
    "trainer.parallel_groups": "parallel.mesh",
    "utils": "utils.misc", "trainer.flops_counter": "flops",
}


def _resolve(fullname: str):
    rest = fullname[len(_PREFIX):]
    for cand in (_MODULES.get(rest), rest):
        if cand is None:
            continue
        try:
            return importlib.import_module(f"arctictraining_b200.{cand}")
        except ImportError:
            continue
    return None


class _AliasFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(_PREFIX):
            return None
        module = _resolve(fullname)
        if module is None:
            return None
        return importlib.machinery.ModuleSpec(fullname, self, is_package=hasattr(module, "__path__"))

    def __init__(self):
        self._specs = {}

    def create_module(self, spec):
        module = _resolve(spec.name)  # the very module object of this package: its classes are the registered ones
        self._specs[id(module)] = (getattr(module, "__spec__", None), getattr(module, "__loader__", None))
        return module

    def exec_module(self, module):
        # the import machinery stamped the alias' spec on the shared module object: put its own back, so that
        # relative imports inside it and importlib.reload keep seeing the module's real identity
        spec, loader = self._specs.pop(id(module), (None, None))
        if spec is not None:
            module.__spec__ = spec
            module.__loader__ = loader


if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())
for _name in dir(_impl):
    if not _name.startswith("__"):
        globals().setdefault(_name, getattr(_impl, _name))

if os.environ.get("ATB200_DEEPSPEED_SHIM", "0") == "1":
    # user code that also imports the reference's engine package by name gets stand-ins backed by this package
    from arctictraining_b200.compat import deepspeed_shim as _shim

    _shim.install()
