# SPDX-License-Identifier: Apache-2.0
"""Direct Preference Optimisation trainer.

Behaviour parity: arctic_training/trainer/dpo_trainer.py:50-271 — a policy model and a frozen reference
model (ZeRO-3 sharded when the policy is, otherwise replicated), batches of chosen rows followed by
rejected rows, sigmoid DPO loss with ``beta`` and ``label_smoothing`` (conservative / robust DPO).  The
sequence log-probabilities come from the tiled fused linear-log-prob op (the lm_head GEMM, the softmax
statistics and the label gather run tile by tile), which stands in for the Triton fused DPO loss the
reference can use.
"""

from __future__ import annotations

from typing import Any
from typing import Dict
from typing import Tuple
from typing import Union
from typing import cast

import torch
import torch.nn.functional as F
from pydantic import ValidationInfo
from pydantic import field_validator
from pydantic import model_validator
from typing_extensions import Self

from .. import ops
from ..checkpoint.hf import HFCheckpointEngine
from ..checkpoint.sharded import DSCheckpointEngine
from ..config.model import ModelConfig
from ..config.trainer import TrainerConfig
from ..data.dpo import DPODataFactory
from ..models.factory import HFModelFactory
from ..models.factory import LigerModelFactory
from ..optimizer.adam import CPUAdamOptimizerFactory
from ..optimizer.adam import FusedAdamOptimizerFactory
from ..registry import get_registered_model_factory
from ..scheduler.factory import HFSchedulerFactory
from ..scheduler.factory import WSDSchedulerFactory
from ..tokenizer.factory import FakeTokenizerFactory
from ..tokenizer.factory import HFTokenizerFactory
from .trainer import Trainer
from .utils import to_device


def get_logprobs(logits: torch.Tensor, labels: torch.Tensor, ignore_label_index: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Sum of label log-probabilities per row and number of unmasked labels, from full logits."""
    if logits.shape[:-1] != labels.shape:
        raise ValueError(f"Logits {logits.shape[:-1]} and labels {labels.shape} must have the same leading shape.")
    labels = labels[:, 1:].clone()
    logits = logits[:, :-1, :]
    mask = labels != ignore_label_index
    labels[~mask] = 0
    per_token = torch.gather(logits.log_softmax(-1), dim=2, index=labels.unsqueeze(2)).squeeze(2)
    return (per_token * mask).sum(-1), mask.sum(-1)


class DPOTrainerConfig(TrainerConfig):
    ref_model: ModelConfig
    """ Reference model (frozen); provides the baseline log-likelihoods. """

    beta: float = 0.1
    """ Strength of the pull towards the reference model. """

    ignore_label_index: int = -100
    """ Label value that is ignored. """

    label_smoothing: float = 0.0
    """ Conservative-DPO label smoothing in [0, 0.5). """

    reference_model_deepspeed: Dict[str, Any] = {}
    """ Engine config of the reference model (derived; must not be given). """

    @field_validator("ref_model", mode="before")
    @classmethod
    def _init_ref_model(cls, v: Union[Dict, ModelConfig], info: ValidationInfo) -> ModelConfig:
        return cast(ModelConfig, cls._subconfig(v, info, get_registered_model_factory, "ref_model_factory"))

    @model_validator(mode="after")
    def _dpo_batch_sizes(self) -> Self:
        # a micro batch holds the chosen and the rejected rows
        self.deepspeed["train_micro_batch_size_per_gpu"] = int(self.micro_batch_size * 2)
        self.deepspeed["train_batch_size"] = int(self.micro_batch_size * self.gradient_accumulation_steps * self.world_size * 2)
        return self

    @model_validator(mode="after")
    def _build_ref_engine_config(self) -> Self:
        if self.reference_model_deepspeed:
            raise ValueError("The reference model's engine config is derived from the main one and must not be given.")
        stage = 3 if self.deepspeed["zero_optimization"].get("stage") == 3 else 0
        object.__setattr__(self, "reference_model_deepspeed", dict(
            train_batch_size=self.deepspeed["train_batch_size"],
            train_micro_batch_size_per_gpu=self.deepspeed["train_micro_batch_size_per_gpu"],
            steps_per_print=self.deepspeed["steps_per_print"],
            zero_optimization=dict(stage=stage, stage3_param_persistence_threshold=1e4),
            bfloat16=dict(enabled=True),
            gradient_clipping=1.0, prescale_gradients=False, wall_clock_breakdown=False,
        ))
        return self


def init_ref_model(self: "DPOTrainer") -> None:
    factory = self.config.ref_model.factory(trainer=self, model_config=self.config.ref_model)
    ref = factory()
    for p in ref.parameters():
        p.requires_grad_(False)
    ref.eval()
    self._configure_model(ref)
    from ..engine import TrainingEngine

    self.ref_model = TrainingEngine(ref, None, None, self.config.reference_model_deepspeed, training=False)


class DPOTrainer(Trainer):
    name = "dpo"
    config: DPOTrainerConfig
    data_factory: DPODataFactory
    model_factory: Union[HFModelFactory, LigerModelFactory]
    ref_model_factory: Union[HFModelFactory, LigerModelFactory]
    checkpoint_engine: Union[DSCheckpointEngine, HFCheckpointEngine]
    optimizer_factory: Union[FusedAdamOptimizerFactory, CPUAdamOptimizerFactory]
    scheduler_factory: Union[HFSchedulerFactory, WSDSchedulerFactory]
    tokenizer_factory: Union[HFTokenizerFactory, FakeTokenizerFactory]

    callbacks = [("post-init", init_ref_model)]

    def sequence_logprobs(self, model, batch: Dict[str, torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
        """Sum of completion log-probabilities per row, through the tiled fused op when the model is native."""
        labels = batch["labels"]
        ignore = self.config.ignore_label_index
        module = model.module if hasattr(model, "module") else model
        if hasattr(module, "lm_head") and hasattr(module, "model") and hasattr(module, "build_context"):
            out = model(input_ids=batch["input_ids"], attention_mask=batch.get("attention_mask"), use_cache=False,
                        labels=None, shift_labels=None, return_logits=False, hidden_only=True)
            hidden = out.hidden_states
            shifted = F.pad(labels[:, 1:], (0, 1), value=ignore)
            if ignore != ops.IGNORE_INDEX:
                shifted = shifted.masked_fill(shifted == ignore, ops.IGNORE_INDEX)
            per_tok = ops.fused_linear_logprobs(hidden, module.lm_head.weight, shifted)
            return per_tok.sum(-1), (shifted != ops.IGNORE_INDEX).sum(-1)
        out = model(input_ids=batch["input_ids"], attention_mask=batch.get("attention_mask"), use_cache=False)
        return get_logprobs(out.logits.float(), labels, ignore)

    def forward_model(self, batch):
        return self.sequence_logprobs(self.model, batch)

    def forward_reference_model(self, batch):
        with torch.no_grad():
            lp, n = self.sequence_logprobs(self.ref_model, batch)
        return lp.detach(), n.detach()

    def dpo_loss(self, logprobs: torch.Tensor, ref_logprobs: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """``-log sigmoid(beta * ((pi_w - pi_l) - (ref_w - ref_l)))`` with optional label smoothing; also
        returns the implicit rewards of the chosen and rejected completions."""
        b = logprobs.size(0) // 2
        pi_w, pi_l = logprobs[:b], logprobs[b:]
        ref_w, ref_l = ref_logprobs[:b], ref_logprobs[b:]
        margin = (pi_w - pi_l) - (ref_w - ref_l)
        beta, eps = self.config.beta, self.config.label_smoothing
        losses = -F.logsigmoid(beta * margin) * (1 - eps) - F.logsigmoid(-beta * margin) * eps
        return losses, beta * (pi_w - ref_w).detach(), beta * (pi_l - ref_l).detach()

    def loss(self, batch) -> torch.Tensor:
        batch = to_device(batch, self.device)
        ref_lp, _ = self.forward_reference_model(batch)
        lp, _ = self.forward_model(batch)
        losses, _, _ = self.dpo_loss(lp, ref_lp)
        return losses.mean()
