# SPDX-License-Identifier: Apache-2.0
"""``tokenizer:`` section.  Parity: arctic_training/config/tokenizer.py:32-44."""

from __future__ import annotations

from pathlib import Path
from typing import TYPE_CHECKING
from typing import Any
from typing import Dict
from typing import Optional
from typing import Type
from typing import Union

from pydantic import Field

from ..registry import get_registered_tokenizer_factory
from .base import BaseConfig

if TYPE_CHECKING:
    from ..tokenizer.factory import TokenizerFactory


class TokenizerConfig(BaseConfig):
    type: str = ""
    """ Tokenizer factory type. Defaults to the first ``tokenizer_factory`` hint of the trainer. """

    name_or_path: Optional[Union[str, Path]] = ""
    """ Tokenizer name or directory; defaults to ``model.name_or_path``. """

    tokenize_kwargs: Dict[str, Any] = Field(default_factory=dict)
    """ Extra keyword arguments handed to the tokenizer call by the data factories. """

    @property
    def factory(self) -> Type["TokenizerFactory"]:
        return get_registered_tokenizer_factory(name=self.type)
