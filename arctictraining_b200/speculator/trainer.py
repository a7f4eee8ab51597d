# SPDX-License-Identifier: Apache-2.0
"""Trainers, model factories and checkpoint engines for speculative-decoding draft heads.

Registered names match the reference projects: ``arctic-lstm-speculator``
(projects/arctic_lstm_speculator/train.py:40-231) and ``spec-decode`` (projects/mlp_speculator/train.py:43-480).
The base model is frozen and run without gradient; the speculator reads its final hidden states and is trained with
teacher forcing: head ``i`` at position ``t`` predicts token ``t + i + 2`` given the true tokens up to ``t + i + 1``.
The per-head losses are computed with the tiled fused linear-cross-entropy op, so the
``heads x tokens x vocabulary`` logits of the reference are never materialised.  The checkpoint engines write the
speculator alone as ``pytorch_model.bin`` + ``config.json`` (gathering ZeRO-3 shards through the engine).
"""

from __future__ import annotations

import os
from typing import Any
from typing import Dict
from typing import Union

import torch
import torch.distributed as dist
from pydantic import model_validator
from typing_extensions import Self

from .. import ops
from ..checkpoint.engine import CheckpointEngine
from ..checkpoint.sharded import DSCheckpointEngine
from ..config.model import ModelConfig
from ..config.trainer import TrainerConfig
from ..data.sft import SFTDataFactory
from ..logging import logger
from ..models.factory import HFModelFactory
from ..trainer.sft import SFTTrainer
from ..trainer.utils import to_device
from .modules import MLPSpeculatorConfig
from .modules import Speculator
from .modules import SpeculatorConfig


def _attach(model: torch.nn.Module, spec_cfg: SpeculatorConfig, train_heads: bool, ckpt: bool) -> torch.nn.Module:
    base_param = next(model.parameters())
    spec = Speculator(spec_cfg)
    spec.reset_parameters()
    model.speculator = spec.to(base_param.dtype).to(base_param.device)
    if train_heads:
        for p in model.parameters():
            p.requires_grad_(False)
        for p in model.speculator.parameters():
            p.requires_grad_(True)
    model.activation_checkpointing = ckpt
    if hasattr(model, "zero_units"):
        base_units = model.zero_units

        def zero_units():
            return base_units() + [("speculator", [model.speculator], False)]

        model.zero_units = zero_units
    return model


class ArcticLSTMSpeculatorModelConfig(ModelConfig):
    n_speculator_heads: int = 3
    speculator_width: Union[int, str] = "4096"
    proj_dim: Union[int, str] = "4096"
    emb_dim: Union[int, str] = "4096"
    speculator_tie_weights: bool = False
    speculator_scale_input: bool = False
    method: str = "sum_rnn"
    tie_lstm_embs: bool = False


class ArcticLSTMSpeculatorModelFactory(HFModelFactory):
    name = "arctic-lstm-speculator"
    config: ArcticLSTMSpeculatorModelConfig

    def post_create_model_callback(self, model):
        c = self.config
        hidden, vocab = model.lm_head.in_features, model.lm_head.out_features
        spec_cfg = SpeculatorConfig(c.name_or_path, hidden, c.speculator_width, c.proj_dim, c.emb_dim, vocab,
                                    c.n_speculator_heads, tie_weights=c.speculator_tie_weights,
                                    scale_input=c.speculator_scale_input, method=c.method, tie_lstm_embs=c.tie_lstm_embs)
        return _attach(model, spec_cfg, c.n_speculator_heads > 0, not c.disable_activation_checkpoint)


class MLPSpeculatorModelConfig(ModelConfig):
    n_speculator_heads: int = 3
    speculator_width: int = 4096
    speculator_tie_weights: bool = False
    speculator_scale_input: bool = False


class MLPSpeculatorModelFactory(HFModelFactory):
    name = "spec-decode"
    config: MLPSpeculatorModelConfig

    def post_create_model_callback(self, model):
        c = self.config
        hidden, vocab = model.lm_head.in_features, model.lm_head.out_features
        spec_cfg = MLPSpeculatorConfig(c.name_or_path, hidden, c.speculator_width, vocab, c.n_speculator_heads,
                                       tie_weights=c.speculator_tie_weights, scale_input=c.speculator_scale_input)
        return _attach(model, spec_cfg, c.n_speculator_heads > 0, not c.disable_activation_checkpoint)


class ArcticLSTMSpeculatorCheckpointEngine(CheckpointEngine):
    """Writes / reads only the speculator: ``pytorch_model.bin`` + ``config.json`` in ``output_dir``."""

    name = "arctic-lstm-speculator"

    @property
    def latest_checkpoint_exists(self) -> bool:
        return (self.config.output_dir / "pytorch_model.bin").exists()

    def save(self, model) -> None:
        module = model.module if hasattr(model, "module") else model
        # the speculator is a unit of its own that the engine keeps gathered, so its state dict is complete on
        # every rank (tied tensors appear under each of their names, as a plain ``Speculator`` expects)
        full = {k: v.detach().to("cpu").clone() for k, v in module.speculator.state_dict().items()}
        if self.global_rank == 0:
            out = self.config.output_dir
            os.makedirs(out, exist_ok=True)
            torch.save(full, out / "pytorch_model.bin")
            module.speculator.config.save(str(out))
            logger.info(f"saved speculator to {out}")
        if dist.is_initialized():
            dist.barrier()

    def load(self, model) -> None:
        path = self.config.output_dir / "pytorch_model.bin"
        if not path.exists():
            return
        state = torch.load(path, map_location="cpu", weights_only=True)
        module = model.module if hasattr(model, "module") else model
        expected = module.speculator.state_dict().keys()
        assert set(state) == set(expected), "checkpoint has different parameters than the speculator"
        if hasattr(model, "units"):
            for u in model.units:
                with model.gathered_unit(u):
                    for n, p in zip(u.param_names, u.params):
                        if n.startswith("speculator."):
                            p.data.copy_(state[n[len("speculator."):]].to(p.dtype))
                    if any(n.startswith("speculator.") for n in u.param_names):
                        lo = u.group_rank * u.shard_size
                        u.shard.copy_(u.flat[lo : lo + u.shard_size])
                        if u.master is not None:
                            u.master[: u.train_len].copy_(u.shard[: u.train_len].to(u.master.dtype))
        else:
            module.speculator.load_state_dict(state)


class MLPSpeculatorCheckpointEngine(ArcticLSTMSpeculatorCheckpointEngine):
    name = "spec-decode"


def speculator_loss(module: torch.nn.Module, hidden: torch.Tensor, input_ids: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    """Sum over heads of the mean cross-entropy; head ``i`` at position ``t`` is scored against ``labels[t + i + 2]``."""
    spec = module.speculator
    n = spec.n_predict
    states = spec.head_states(hidden[:, : -n - 1, :], input_ids[:, 1:])
    N = states[0].size(1)
    total = hidden.new_zeros((), dtype=torch.float32)
    for i, st in enumerate(states):
        targ = labels[:, i + 2 : N + i + 2]
        loss_sum, cnt = ops.fused_linear_cross_entropy(st, spec.head[i].weight, targ)
        total = total + loss_sum / cnt.clamp(min=1).to(loss_sum.dtype)
    return total


class ArcticLSTMSpeculatorTrainer(SFTTrainer):
    supports_sequence_parallel = False  # the heads predict from whole hidden-state sequences
    name = "arctic-lstm-speculator"
    data_factory: SFTDataFactory
    model_factory: ArcticLSTMSpeculatorModelFactory
    checkpoint_engine: Union[DSCheckpointEngine, ArcticLSTMSpeculatorCheckpointEngine]

    def base_hidden_states(self, inputs: Dict[str, Any]) -> torch.Tensor:
        with torch.no_grad():
            out = self.model(input_ids=inputs["input_ids"], position_ids=inputs.get("position_ids"), hidden_only=True,
                             use_cache=False)
        return out.hidden_states.detach()

    def loss(self, batch) -> torch.Tensor:
        inputs = to_device(batch, self.device)
        inputs.pop("packed_sample_seqlens", None)
        hidden = self.base_hidden_states(inputs)
        return speculator_loss(self.model_unwrapped, hidden, inputs["input_ids"], inputs["labels"])


class MLPSpeculatorTrainerConfig(TrainerConfig):
    gen_train: bool = False
    """ Train on continuations generated on the fly by the base model instead of the dataset's own tokens. """
    gen_train_simple: bool = False
    """ With ``gen_train``: one speculator update per generated batch.  Without it, a batch of ``gen_micro_batch_size``
    prompts is generated at once and the speculator is updated once per ``gen_train_micro_batch_size`` of them. """
    gen_micro_batch_size: int = 384
    gen_train_global_batch_size: int = 2048
    gen_train_micro_batch_size: int = 32
    gen_prompt_length: int = 64
    gen_seq_length: int = 256

    @model_validator(mode="after")
    def _check_gen_train(self) -> Self:
        if self.gen_train and not self.gen_train_simple:
            assert self.gen_micro_batch_size % self.gen_train_micro_batch_size == 0, (
                "gen_micro_batch_size must be divisible by gen_train_micro_batch_size"
            )
            assert self.gen_micro_batch_size % self.micro_batch_size == 0, (
                "gen_micro_batch_size must be a multiple of micro_batch_size"
            )
        elif self.gen_train:
            assert self.gen_train_micro_batch_size == self.gen_micro_batch_size, (
                "gen_train_micro_batch_size must equal gen_micro_batch_size"
            )
        return self


def speculator_loss_on_generated(module: torch.nn.Module, hidden: torch.Tensor, tokens: torch.Tensor) -> torch.Tensor:
    """Loss on sequences the base model generated itself: ``hidden[:, t]`` is the state that produced ``tokens[:, t + 1]``
    and head ``i`` at position ``t`` is scored against ``tokens[:, t + i + 1]`` (the reference's generation losses,
    projects/mlp_speculator/train.py:329-416)."""
    spec = module.speculator
    states = spec.head_states(hidden, tokens[:, :-1])
    N = states[0].size(1)
    total = hidden.new_zeros((), dtype=torch.float32)
    for i, st in enumerate(states):
        targ = tokens[:, i + 1 : N + i + 1]
        loss_sum, cnt = ops.fused_linear_cross_entropy(st[:, : targ.shape[1]], spec.head[i].weight, targ)
        total = total + loss_sum / cnt.clamp(min=1).to(loss_sum.dtype)
    return total


class MLPSpeculatorTrainer(ArcticLSTMSpeculatorTrainer):
    name = "spec-decode"
    config: MLPSpeculatorTrainerConfig
    model_factory: MLPSpeculatorModelFactory
    checkpoint_engine: Union[DSCheckpointEngine, MLPSpeculatorCheckpointEngine]

    @torch.no_grad()
    def generate_continuations(self, prompt_ids: torch.Tensor, new_tokens: int) -> torch.Tensor:
        """Greedy continuation by the frozen base model that re-runs the whole sequence for every token (the oracle of
        the cached generation)."""
        ids = prompt_ids
        for _ in range(new_tokens):
            out = self.model(input_ids=ids, return_logits=True, use_cache=False)
            ids = torch.cat([ids, out.logits[:, -1:].argmax(-1)], dim=1)
        return ids

    @torch.no_grad()
    def generate(self, prompts: torch.Tensor, new_tokens: int, do_sample: bool = True):
        """Sampled (top-k 10) continuation with a key/value cache; returns ``(tokens, hidden states)``."""
        from ..models.generation import generate

        self.model.eval()
        try:
            return generate(self.model_unwrapped, prompts, new_tokens, do_sample=do_sample)
        finally:
            self.model.train()

    def _generated_batch(self, batch, rows: int):
        """Cut the batch's token rows into ``rows`` prompts of ``gen_prompt_length`` tokens, generate ``gen_seq_length``
        tokens after each and keep the generated part with the states that produced it."""
        c = self.config
        inputs = to_device(batch, self.device)
        ids = inputs["input_ids"]
        grow = max(1, rows // ids.shape[0])
        assert c.gen_prompt_length * grow <= ids.shape[1], "the batch is too short for gen_prompt_length x gen_micro_batch_size"
        prompts = ids[:, : c.gen_prompt_length * grow].reshape(ids.shape[0] * grow, c.gen_prompt_length)
        tokens, hidden = self.generate(prompts, c.gen_seq_length)
        n = self.model_unwrapped.speculator.n_predict
        tokens = tokens[:, -c.gen_seq_length :]
        # hidden[:, t] belongs to input position t and predicts token t + 1: the state before the first generated token
        # comes first; the last n states have no complete set of targets
        hidden = hidden[:, -c.gen_seq_length : hidden.shape[1] - n]
        return tokens, hidden.detach()

    def loss(self, batch) -> torch.Tensor:
        if isinstance(batch, dict) and "speculator_input" in batch:
            # speculator-only update on states and tokens that were generated earlier (see step)
            return speculator_loss_on_generated(self.model_unwrapped, batch["speculator_input"], batch["speculator_label"])
        if not self.config.gen_train:
            return super().loss(batch)
        tokens, hidden = self._generated_batch(batch, batch["input_ids"].shape[0])
        return speculator_loss_on_generated(self.model_unwrapped, hidden, tokens)

    def step(self, batch) -> None:
        c = self.config
        if not c.gen_train or c.gen_train_simple:
            return super().step(batch)
        # one generation of gen_micro_batch_size sequences feeds several speculator updates of gen_train_micro_batch_size
        rows = batch["input_ids"].shape[0] * (c.gen_micro_batch_size // c.micro_batch_size)
        tokens, hidden = self._generated_batch(batch, rows)
        mb = min(c.gen_train_micro_batch_size, tokens.shape[0])
        for s in range(0, tokens.shape[0] - mb + 1, mb):
            self.metrics.values.pop("loss", None)  # one loss per update; the last one is reported for the iteration
            super().step({"speculator_input": hidden[s : s + mb], "speculator_label": tokens[s : s + mb]})
