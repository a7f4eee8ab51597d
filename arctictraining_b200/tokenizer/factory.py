# SPDX-License-Identifier: Apache-2.0
"""Tokenizer factories.  Parity: arctic_training/tokenizer/factory.py:35-87, hf_factory.py:23-31; the
``fake`` factory corresponds to the test tokenizer of the embedding project
(projects/arctic_embed/src/arctic_embed/trainer.py:67-71)."""

from __future__ import annotations

from abc import ABC
from abc import abstractmethod
from pathlib import Path
from typing import TYPE_CHECKING
from typing import Any
from typing import Optional

from ..callback.mixin import CallbackMixin
from ..callback.mixin import callback_wrapper
from ..config.tokenizer import TokenizerConfig
from ..registry import RegistryMeta
from ..registry import _validate_class_attribute_set
from ..registry import _validate_class_attribute_type
from ..registry import _validate_class_method
from ..utils.factory_base import TrainerBound
from .fake import FakeTokenizer

if TYPE_CHECKING:
    from ..trainer.trainer import Trainer


class TokenizerFactory(ABC, CallbackMixin, TrainerBound, metaclass=RegistryMeta):
    name: str
    """ Name under which the factory is selected in a recipe (``tokenizer.type``). """

    config: TokenizerConfig
    """ Config class of this factory. """

    @classmethod
    def _validate_subclass(cls) -> None:
        _validate_class_attribute_set(cls, "name")
        _validate_class_attribute_type(cls, "config", TokenizerConfig)
        _validate_class_method(cls, "create_tokenizer", ["self"])

    def __init__(self, trainer: "Trainer", tokenizer_config: Optional[TokenizerConfig] = None) -> None:
        self._trainer = trainer
        self.config = tokenizer_config if tokenizer_config is not None else trainer.config.tokenizer

    def __call__(self) -> Any:
        return self.create_tokenizer()

    @abstractmethod
    @callback_wrapper("create-tokenizer")
    def create_tokenizer(self) -> Any:
        raise NotImplementedError


class HFTokenizerFactory(TokenizerFactory):
    name = "huggingface"

    def create_tokenizer(self) -> Any:
        from ..models.arch import PRESETS

        path = str(self.config.name_or_path)
        if path.lower() in PRESETS or (Path(path) / "fake_tokenizer.json").exists():
            # architecture presets ship no tokenizer files: use the hash tokenizer sized to the vocabulary
            vocab = PRESETS[path.lower()]["vocab_size"] if path.lower() in PRESETS else None
            return FakeTokenizer(vocab) if vocab else FakeTokenizer.from_pretrained(path)
        from transformers import AutoTokenizer

        tok = AutoTokenizer.from_pretrained(path)
        if tok.pad_token is None:
            tok.pad_token = tok.eos_token
        return tok


class FakeTokenizerFactory(TokenizerFactory):
    name = "fake"

    def create_tokenizer(self) -> Any:
        from ..models.arch import PRESETS

        path = str(self.config.name_or_path).lower()
        return FakeTokenizer(PRESETS[path]["vocab_size"]) if path in PRESETS else FakeTokenizer()
