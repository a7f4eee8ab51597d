# SPDX-License-Identifier: Apache-2.0
"""MoBA project: the SwiftKV-free variant of the reference's trainer (projects/moba_attention/train.py:23-61) — an SFT
trainer whose model factory swaps the attention core for Mixture-of-Block-Attention."""

from typing import Union

from arctictraining_b200.attention.moba import MoBAContext
from arctictraining_b200.checkpoint.hf import HFCheckpointEngine
from arctictraining_b200.checkpoint.sharded import DSCheckpointEngine
from arctictraining_b200.config.model import ModelConfig
from arctictraining_b200.models.factory import HFModelFactory
from arctictraining_b200.trainer.sft import SFTTrainer


class MoBAModelConfig(ModelConfig):
    moba_chunk_size: int = 4096
    """ Key block size. """
    moba_topk: int = 8
    """ Blocks each query attends to (its own block included). """


class MoBAModelFactory(HFModelFactory):
    name = "moba"
    config: MoBAModelConfig

    def post_create_model_callback(self, model):
        model = super().post_create_model_callback(model)
        model.sp_context = MoBAContext(self.config.moba_chunk_size, self.config.moba_topk)
        model._keep_sp_context = True
        return model


class MoBATrainer(SFTTrainer):
    name = "moba"
    model_factory: MoBAModelFactory
    checkpoint_engine: Union[DSCheckpointEngine, HFCheckpointEngine]

    def _configure_model(self, model) -> None:
        keep = getattr(model, "sp_context", None)
        super()._configure_model(model)
        if getattr(model, "_keep_sp_context", False):
            model.sp_context = keep
