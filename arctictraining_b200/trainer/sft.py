# SPDX-License-Identifier: Apache-2.0
"""Supervised fine-tuning and causal-LM trainers.

Behaviour parity: arctic_training/trainer/sft_trainer.py:38-166 and causal_trainer.py:31-40.  The native
model always computes the loss with the tiled fused linear-cross-entropy op, so the three code paths of
the reference (plain HF loss, Liger fused loss, tiled logits+loss under sequence parallelism) collapse
into one.  Under sequence parallelism the batch carries ``shift_labels`` and the loss is the
token-weighted mean over the group, identical on every rank.
"""

from __future__ import annotations

from typing import Any
from typing import Dict
from typing import Union

import torch

from ..checkpoint.engine import CheckpointEngine
from ..checkpoint.hf import HFCheckpointEngine
from ..checkpoint.sharded import DSCheckpointEngine
from ..config.trainer import TrainerConfig
from ..data.causal import CausalDataFactory
from ..data.sft import SFTDataFactory
from ..models.factory import HFModelFactory
from ..models.factory import LigerModelFactory
from ..optimizer.adam import CPUAdamMoEOptimizerFactory
from ..optimizer.adam import CPUAdamOptimizerFactory
from ..optimizer.adam import FusedAdamMoEOptimizerFactory
from ..optimizer.adam import FusedAdamOptimizerFactory
from ..scheduler.factory import HFSchedulerFactory
from ..scheduler.factory import WSDSchedulerFactory
from ..tokenizer.factory import FakeTokenizerFactory
from ..tokenizer.factory import HFTokenizerFactory
from .trainer import Trainer
from .utils import to_device


class SFTTrainer(Trainer):
    name = "sft"
    supports_sequence_parallel = True
    config: TrainerConfig
    data_factory: SFTDataFactory
    model_factory: Union[HFModelFactory, LigerModelFactory]
    checkpoint_engine: Union[DSCheckpointEngine, HFCheckpointEngine]
    optimizer_factory: Union[
        FusedAdamOptimizerFactory, CPUAdamOptimizerFactory, FusedAdamMoEOptimizerFactory, CPUAdamMoEOptimizerFactory
    ]
    scheduler_factory: Union[HFSchedulerFactory, WSDSchedulerFactory]
    tokenizer_factory: Union[HFTokenizerFactory, FakeTokenizerFactory]

    def loss(self, batch: Dict[str, Any]) -> torch.Tensor:
        batch = to_device(batch, self.device)
        batch.pop("packed_sample_seqlens", None)
        sp = self.config.sequence_parallel_size
        if sp > 1:
            if "labels" in batch:
                raise ValueError("under sequence parallelism the batch must carry `shift_labels`, not `labels`")
            if "shift_labels" not in batch:
                raise ValueError("`shift_labels` is missing from the batch (is the dataloader wrapped for sequence parallelism?)")
        if sp > 1 and getattr(self, "hf_ulysses", None) is not None:
            return self._library_model_sp_loss(batch)
        if sp == 1 and "labels" in batch and getattr(self.model_unwrapped, "_atb_fused_loss", False):
            return self._library_model_fused_loss(batch)
        outputs = self.model(**batch, use_cache=False)
        if sp == 1:
            return outputs.loss
        if getattr(outputs, "loss_sum", None) is None:
            raise ValueError("sequence parallelism needs a model that reports `loss_sum` and `num_tokens`")
        loss = self.sp_context.aggregate_loss(outputs.loss_sum, outputs.num_tokens)
        if getattr(outputs, "aux_loss", None) is not None:
            loss = loss + outputs.aux_loss
        return loss


    def _library_model_fused_loss(self, batch: Dict[str, Any]) -> torch.Tensor:
        """A ``transformers`` model created with ``model.type: liger``: hidden states from the model body, then the tiled
        fused output projection + cross-entropy of this package (mean over target tokens, as the library computes)."""
        from .. import ops

        model = self.model_unwrapped
        if hasattr(model, "get_base_model"):  # an adapter wrapper of the peft package around the causal-LM model
            model = model.get_base_model()
        body = getattr(model, getattr(model, "base_model_prefix", "model"))
        labels = batch.pop("labels")
        shift_labels = torch.nn.functional.pad(labels[..., 1:], (0, 1), value=-100)
        with self.model._timed("forward"), self.model.autocast():
            hidden = body(**batch, use_cache=False).last_hidden_state
            loss_sum, num_tokens = ops.fused_linear_cross_entropy(hidden, model.get_output_embeddings().weight, shift_labels)
        return loss_sum / num_tokens.clamp(min=1)

    def _library_model_sp_loss(self, batch: Dict[str, Any]) -> torch.Tensor:
        """A ``transformers`` model under sequence parallelism: hidden states of this rank's slice from the model body,
        output projection and cross-entropy chunk by chunk, then the token-weighted mean over the group."""
        from ..parallel.ulysses_hf import chunked_causal_lm_loss_sum

        model = self.model_unwrapped
        if hasattr(model, "get_base_model"):  # an adapter wrapper of the peft package around the causal-LM model
            model = model.get_base_model()
        body = getattr(model, getattr(model, "base_model_prefix", "model"), None)
        head = model.get_output_embeddings() if hasattr(model, "get_output_embeddings") else None
        if body is None or head is None:
            raise ValueError(f"{type(model).__name__} does not expose a model body and an output projection")
        shift_labels = batch.pop("shift_labels")
        with self.model._timed("forward"), self.model.autocast():
            hidden = body(**batch, use_cache=False).last_hidden_state
            loss_sum, num_tokens = chunked_causal_lm_loss_sum(head, hidden, shift_labels)
        return self.sp_context.aggregate_loss(loss_sum, num_tokens)


class CausalTrainer(SFTTrainer):
    name = "causal"
    data_factory: CausalDataFactory
