# SPDX-License-Identifier: Apache-2.0
from .factory import FakeTokenizerFactory
from .factory import HFTokenizerFactory
from .factory import TokenizerFactory
from .fake import FakeTokenizer

__all__ = ["FakeTokenizerFactory", "HFTokenizerFactory", "TokenizerFactory", "FakeTokenizer"]
