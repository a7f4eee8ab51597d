# SPDX-License-Identifier: Apache-2.0
"""``model:`` section of a recipe.  Parity: arctic_training/config/model.py:35-98."""

from __future__ import annotations

from pathlib import Path
from typing import TYPE_CHECKING
from typing import Any
from typing import Dict
from typing import Optional
from typing import Type
from typing import Union

from pydantic import Field
from pydantic import field_validator

from ..registry import get_registered_model_factory
from .base import BaseConfig
from .enums import DType

if TYPE_CHECKING:
    from ..models.factory import ModelFactory

_ATTN_IMPLS = ("native", "sdpa", "flash_attention_2", "flash_attention_3", "eager")


class ModelConfig(BaseConfig):
    type: str = ""
    """ Model factory type. """

    name_or_path: Union[str, Path]
    """ Hugging Face style model directory (``config.json`` + safetensors), hub name, or a built-in
    architecture preset such as ``llama-3.1-8b`` (random initialisation). """

    dtype: DType = DType.BF16
    """ Data type of the model weights. """

    save_name: Optional[str] = None
    """ Name to use when saving the model. """

    attn_implementation: str = "sdpa"
    """ Core attention: ``native`` (this framework's sm_100a kernel), ``sdpa``, ``flash_attention_2``/``_3``, ``eager``. """

    disable_activation_checkpoint: bool = False
    """ Disable per-layer activation checkpointing. """

    peft_config: Optional[Dict[str, Any]] = None
    """ Parameter-efficient fine-tuning: ``{peft_type: LORA, r: 8, lora_alpha: 16, target_modules: [...]}``. """

    hf_config_kwargs: Dict[str, Any] = Field(default_factory=dict)
    """ Overrides applied on top of the architecture config (e.g. ``num_hidden_layers: 2``). """

    @property
    def factory(self) -> Type["ModelFactory"]:
        return get_registered_model_factory(name=self.type)

    @property
    def peft_config_obj(self) -> Any:
        """The adapter settings as a config object of the ``peft`` package (needs that package); without the package,
        a plain namespace with the same fields, which is what the built-in LoRA of the native models reads."""
        if self.peft_config is None:
            raise ValueError("No PEFT config specified.")
        conf = dict(self.peft_config)
        conf["peft_type"] = str(conf["peft_type"]).upper()
        try:
            import peft
        except ImportError:
            from types import SimpleNamespace

            return SimpleNamespace(**conf)
        return peft.get_peft_config(conf)

    @field_validator("peft_config", mode="before")
    @classmethod
    def _check_peft(cls, value: Optional[Dict]) -> Optional[Dict]:
        if value is not None:
            if "peft_type" not in value:
                raise ValueError("No 'peft_type' specified in PEFT config.")
            from ..models.peft import SUPPORTED_PEFT_TYPES
            from ..models.peft import library_peft_types

            valid = list(SUPPORTED_PEFT_TYPES) + [t for t in library_peft_types() if t not in SUPPORTED_PEFT_TYPES]
            if str(value["peft_type"]).upper() not in valid:
                raise ValueError(f"PEFT type {value['peft_type']} config not found. Valid PEFT types are: {valid}")
        return value

    @field_validator("attn_implementation", mode="after")
    @classmethod
    def _check_attn(cls, value: str) -> str:
        if value not in _ATTN_IMPLS:
            raise ValueError(f"attn_implementation must be one of {_ATTN_IMPLS}, got {value!r}")
        return value
