# SPDX-License-Identifier: Apache-2.0
"""MoBA project: SwiftKV self-distillation in which every attention call is Mixture-of-Block-Attention.

Parity: projects/moba_attention/train.py:23-61 of the reference — ``MoBATrainer`` is the SwiftKV trainer, its model
factory is the SwiftKV factory plus the MoBA settings (``moba_chunk_size``, ``moba_topk``); the reference patches the
attention library call globally, here the model's attention core is swapped for :class:`MoBAContext` (teacher and
student passes both go through it).  ``moba-sft`` is the same attention under plain supervised fine-tuning.
"""

import importlib.util
import sys
from pathlib import Path
from typing import Union

from arctictraining_b200.attention.moba import MoBAContext
from arctictraining_b200.checkpoint.hf import HFCheckpointEngine
from arctictraining_b200.checkpoint.sharded import DSCheckpointEngine
from arctictraining_b200.config.model import ModelConfig
from arctictraining_b200.models.factory import HFModelFactory
from arctictraining_b200.trainer.sft import SFTTrainer


def _swiftkv_module():
    """The SwiftKV project's ``train.py`` (a sibling folder), imported once under a fixed module name."""
    name = "atb200_projects_swiftkv_train"
    if name not in sys.modules:
        path = Path(__file__).resolve().parent.parent / "swiftkv" / "train.py"
        for mod in list(sys.modules.values()):  # already imported as a recipe's ``code:`` file?
            if getattr(mod, "__file__", None) and Path(mod.__file__).resolve() == path and hasattr(mod, "SwiftKVTrainer"):
                sys.modules[name] = mod
                break
        else:
            spec = importlib.util.spec_from_file_location(name, path)
            module = importlib.util.module_from_spec(spec)
            sys.modules[name] = module
            spec.loader.exec_module(module)
    return sys.modules[name]


_swiftkv = _swiftkv_module()


def _install_moba(model, chunk_size: int, topk: int):
    model.sp_context = MoBAContext(chunk_size, topk)
    model._keep_sp_context = True
    return model


class _KeepsAttentionCore:
    """The trainer resets ``model.sp_context`` when it configures the model; MoBA has to survive that."""

    def _configure_model(self, model) -> None:
        keep = getattr(model, "sp_context", None)
        super()._configure_model(model)
        if getattr(model, "_keep_sp_context", False):
            model.sp_context = keep


# ------------------------------------------------------------------------------------------------ distillation (reference)
class MoBAModelConfig(_swiftkv.SwiftKVModelConfig):
    key_value_group_size: int = 1
    moba_chunk_size: int = 4096
    """ Key block size. """
    moba_topk: int = 8
    """ Blocks each query attends to (its own block included). """


class MoBAModelFactory(_swiftkv.SwiftKVModelFactory):
    name = "moba"
    config: MoBAModelConfig

    def post_create_config_callback(self, hf_config):
        hf_config = super().post_create_config_callback(hf_config)
        hf_config["moba_chunk_size"] = self.config.moba_chunk_size
        hf_config["moba_topk"] = self.config.moba_topk
        return hf_config

    def post_create_model_callback(self, model):
        model = super().post_create_model_callback(model)
        return _install_moba(model, self.config.moba_chunk_size, self.config.moba_topk)


class MoBATrainerConfig(_swiftkv.SwiftKVTrainerConfig):
    pass


class MoBATrainer(_KeepsAttentionCore, _swiftkv.SwiftKVTrainer):
    name = "moba"
    config: MoBATrainerConfig
    model_factory: MoBAModelFactory
    checkpoint_engine: Union[DSCheckpointEngine, HFCheckpointEngine]


# ------------------------------------------------------------------------------------------------ plain SFT with MoBA
class MoBASFTModelConfig(ModelConfig):
    moba_chunk_size: int = 4096
    moba_topk: int = 8


class MoBASFTModelFactory(HFModelFactory):
    name = "moba-sft"
    config: MoBASFTModelConfig

    def post_create_model_callback(self, model):
        model = super().post_create_model_callback(model)
        return _install_moba(model, self.config.moba_chunk_size, self.config.moba_topk)


class MoBASFTTrainer(_KeepsAttentionCore, SFTTrainer):
    name = "moba-sft"
    model_factory: MoBASFTModelFactory
    checkpoint_engine: Union[DSCheckpointEngine, HFCheckpointEngine]
