# SPDX-License-Identifier: Apache-2.0
"""Model factories.  Parity: arctic_training/model/factory.py:36-97, hf_factory.py:25-89,
liger_factory.py:24-69.

``huggingface`` builds this framework's native decoder for the supported families (Llama, Qwen2, Qwen3,
Qwen3-MoE, DeepSeek-V2) — weights come from an HF-layout directory, or are random when the recipe names a built-in
preset or overrides ``num_hidden_layers`` — and falls back to ``transformers.AutoModelForCausalLM`` for
other architectures.  ``liger`` is kept as a recipe-compatible alias: the fused kernels it stands for
(RMSNorm, RoPE, SwiGLU, fused linear cross-entropy) are always on in the native model.
"""

from __future__ import annotations

import os
from abc import ABC
from abc import abstractmethod
from pathlib import Path
from typing import TYPE_CHECKING
from typing import Any
from typing import Optional

import torch

from ..callback.mixin import CallbackMixin
from ..callback.mixin import callback_wrapper
from ..config.model import ModelConfig
from ..logging import logger
from ..registry import RegistryMeta
from ..registry import _validate_class_attribute_set
from ..registry import _validate_class_attribute_type
from ..registry import _validate_class_method
from .arch import ArchConfig
from .arch import load_arch_config

if TYPE_CHECKING:
    from ..trainer.trainer import Trainer

NATIVE_MODEL_TYPES = ("llama", "qwen2", "qwen3", "qwen3_moe", "mistral", "deepseek_v2")


class ModelFactory(ABC, CallbackMixin, metaclass=RegistryMeta):
    """Base class for model creation."""

    name: str
    """ Name under which the factory is selected in a recipe (``model.type``). """

    config: ModelConfig
    """ Config class of this factory. """

    @classmethod
    def _validate_subclass(cls) -> None:
        _validate_class_attribute_set(cls, "name")
        _validate_class_attribute_type(cls, "config", ModelConfig)
        _validate_class_method(cls, "create_config", ["self"])
        _validate_class_method(cls, "create_model", ["self", "model_config"])

    def __init__(self, trainer: "Trainer", model_config: Optional[ModelConfig] = None) -> None:
        self._trainer = trainer
        self.config = model_config if model_config is not None else trainer.config.model

    def __call__(self) -> torch.nn.Module:
        return self.create_model(model_config=self.create_config())

    @property
    def trainer(self) -> "Trainer":
        return self._trainer

    @property
    def device(self):
        device = getattr(self.trainer, "device", None)
        if device is None:  # a stand-in trainer object (tests, scripts that only build a model)
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        return device

    @property
    def world_size(self) -> int:
        return getattr(self.trainer, "world_size", int(os.getenv("WORLD_SIZE", 1)))

    @property
    def global_rank(self) -> int:
        return getattr(self.trainer, "global_rank", int(os.getenv("RANK", 0)))

    @abstractmethod
    @callback_wrapper("create-config")
    def create_config(self) -> Any:
        raise NotImplementedError

    @abstractmethod
    @callback_wrapper("create-model")
    def create_model(self, model_config) -> torch.nn.Module:
        raise NotImplementedError


class HFModelFactory(ModelFactory):
    name = "huggingface"
    library_kernels = False  # put this package's ops into a model that is built through the transformers library
    model_cls = None  # set lazily to CausalLM; subclasses override

    def create_config(self) -> ArchConfig:
        base = load_arch_config(self.config.name_or_path)
        cfg = load_arch_config(self.config.name_or_path, self.config.hf_config_kwargs)
        layers_override = self.config.hf_config_kwargs.get("num_hidden_layers")
        self.using_random_model = base.get("_source") == "preset" or (
            layers_override is not None and layers_override != base.get("num_hidden_layers")
        )
        return cfg

    def _native_class(self, model_config=None):
        from .causal_lm import CausalLM

        if self.model_cls is None and model_config is not None and model_config.get("model_type") == "deepseek_v2":
            from .deepseek import DeepseekV2ForCausalLM

            return DeepseekV2ForCausalLM
        return self.model_cls or CausalLM

    def create_model(self, model_config) -> torch.nn.Module:
        dtype = self.config.dtype.value if hasattr(self.config.dtype, "value") else self.config.dtype
        if model_config.get("model_type") not in NATIVE_MODEL_TYPES:
            return self._create_transformers_model(model_config, dtype)
        device = self.device
        from ..moe.layer import expert_parallel_layout

        groups = getattr(self.trainer, "groups", None)
        use_ep = groups is not None and groups.ep_size > 1 and getattr(self.trainer.config, "arctic_moe", False) not in (False, None)
        layout = expert_parallel_layout(groups.ep_size, groups.ep_rank, groups.ep_group) if use_ep else expert_parallel_layout(1, 0, None)
        with torch.device(device), layout:
            model = self._native_class(model_config)(model_config, dtype=dtype)
        model.attn_impl = self.config.attn_implementation
        if self.using_random_model:
            model.init_weights(seed=getattr(self.trainer.config, "seed", 42) if self.trainer is not None else 42)
        else:
            from .hf_io import load_pretrained_into

            load_pretrained_into(model, Path(str(self.config.name_or_path)), model_config)
        return model

    def _create_transformers_model(self, model_config, dtype) -> torch.nn.Module:
        from transformers import AutoConfig
        from transformers import AutoModelForCausalLM

        hf_cfg = AutoConfig.from_pretrained(self.config.name_or_path)
        for k, v in self.config.hf_config_kwargs.items():
            setattr(hf_cfg, k, v)
        attn = self.config.attn_implementation if self.config.attn_implementation != "native" else "sdpa"
        if self.using_random_model:
            model = AutoModelForCausalLM.from_config(hf_cfg, attn_implementation=attn, dtype=dtype)
        else:
            model = AutoModelForCausalLM.from_pretrained(
                self.config.name_or_path, config=hf_cfg, attn_implementation=attn, dtype=dtype
            )
        model = model.to(self.device)
        if self.library_kernels:
            from .hf_kernels import apply_kernels_to_hf_model

            counts = apply_kernels_to_hf_model(model)
            logger.info(f"library model: {counts['rms_norm']} RMSNorm modules on the own kernel, fused loss "
                        f"{'on' if model._atb_fused_loss else 'off'}")
        return model

    def post_create_model_callback(self, model):
        if self.config.peft_config is not None:
            from .causal_lm import CausalLM
            from .peft import SUPPORTED_PEFT_TYPES
            from .peft import apply_library_peft
            from .peft import apply_lora

            kind = str(self.config.peft_config["peft_type"]).upper()
            if isinstance(model, CausalLM) or getattr(model, "model", None).__class__.__module__.startswith("arctictraining_b200"):
                if kind not in SUPPORTED_PEFT_TYPES:
                    raise ValueError(f"PEFT type {kind} is not available on the native models (supported: {SUPPORTED_PEFT_TYPES})")
                trainable, total = apply_lora(model, self.config.peft_config)
            else:
                model = apply_library_peft(model, self.config.peft_config)
                trainable = sum(p.numel() for p in model.parameters() if p.requires_grad)
                total = sum(p.numel() for p in model.parameters())
            logger.info(f"Applied PEFT config: total params {total}, trainable {trainable} ({100 * trainable / total:.2f}%)")
        model.activation_checkpointing = not self.config.disable_activation_checkpoint
        if hasattr(model, "gradient_checkpointing_enable") and not self.config.disable_activation_checkpoint:
            # kept for parity of the model's flags; the engine checkpoints (and, when asked, offloads) the inputs of
            # the decoder layers itself, and a layer is computed twice per step, not three times (tested)
            model.gradient_checkpointing_enable()
        return model


class LigerModelFactory(HFModelFactory):
    """Recipe name of the reference for "use the fused kernels".  Own architectures always do; a model of the
    transformers library gets this package's RMSNorm kernel and the fused output-projection + cross-entropy loss."""

    name = "liger"
    library_kernels = True
