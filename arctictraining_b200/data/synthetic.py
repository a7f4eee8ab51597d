# SPDX-License-Identifier: Apache-2.0
"""Synthetic data sources: seeded uniform token ids, no files and no network.

``synthetic`` yields already tokenised samples (``input_ids``/``labels``/``attention_mask``; set
``process: false`` is implied) with lengths drawn uniformly from ``[min_length, max_length]`` and the first
``prompt_fraction`` of every sample masked with -100, which is the shape of data the benchmarks and the
plumbing tests use.  ``synthetic_messages`` yields chat ``messages`` so that the whole tokenisation path
can be exercised with the hash tokenizer.  ``synthetic_dpo`` yields prompt/chosen/rejected triples.
The reference has no such source; its tests download small hub datasets instead
(tests/data/test_sft_factory.py:24-110).
"""

from __future__ import annotations

from typing import Optional

import numpy as np
from pydantic import Field
from pydantic import model_validator
from typing_extensions import Self

from ..config.data import DataSourceConfig
from .source import DataSource

IGNORE_INDEX = -100


class SyntheticSourceConfig(DataSourceConfig):
    name_or_path: str = "synthetic"
    num_samples: int = Field(default=64, ge=1)
    """ Number of samples to generate. """
    min_length: int = Field(default=128, ge=2)
    max_length: int = Field(default=128, ge=2)
    """ Sample lengths are uniform in ``[min_length, max_length]``. """
    vocab_size: Optional[int] = None
    """ Ids are uniform in ``[low_id, vocab_size)``; defaults to the tokenizer's vocabulary size. """
    low_id: int = 8
    prompt_fraction: float = Field(default=0.5, ge=0.0, le=1.0)
    """ Leading fraction of each sample whose labels are masked. """
    seed: int = 1234
    process: bool = False

    @model_validator(mode="after")
    def _ordered(self) -> Self:
        assert self.min_length <= self.max_length, "min_length must not exceed max_length"
        return self


class SyntheticDataSource(DataSource):
    name = "synthetic"
    config: SyntheticSourceConfig

    def load(self, config: SyntheticSourceConfig, split: str):
        from datasets import Dataset

        vocab = config.vocab_size or len(self.trainer.tokenizer)
        rng = np.random.default_rng(config.seed + (0 if split == "train" else 7919))
        lens = rng.integers(config.min_length, config.max_length + 1, size=config.num_samples)
        ids, labels, masks = [], [], []
        for n in lens:
            row = rng.integers(config.low_id, vocab, size=int(n), dtype=np.int64)
            lab = row.copy()
            lab[: int(n * config.prompt_fraction)] = IGNORE_INDEX
            ids.append(row.tolist())
            labels.append(lab.tolist())
            masks.append([1] * int(n))
        return Dataset.from_dict({"input_ids": ids, "labels": labels, "attention_mask": masks})


class SyntheticMessagesConfig(DataSourceConfig):
    name_or_path: str = "synthetic_messages"
    num_samples: int = Field(default=64, ge=1)
    turns: int = Field(default=2, ge=1)
    words_per_message: int = Field(default=24, ge=1)
    seed: int = 1234


class SyntheticMessagesSource(DataSource):
    name = "synthetic_messages"
    config: SyntheticMessagesConfig

    def load(self, config: SyntheticMessagesConfig, split: str):
        from datasets import Dataset

        rng = np.random.default_rng(config.seed + (0 if split == "train" else 7919))

        def sentence() -> str:
            return " ".join(f"w{int(i)}" for i in rng.integers(0, 5000, size=config.words_per_message))

        rows = []
        for _ in range(config.num_samples):
            msgs = []
            for _ in range(config.turns):
                msgs.append({"role": "user", "content": sentence()})
                msgs.append({"role": "assistant", "content": sentence()})
            rows.append(msgs)
        return Dataset.from_dict({"messages": rows})


class SyntheticDPOSource(DataSource):
    name = "synthetic_dpo"
    config: SyntheticMessagesConfig

    def load(self, config: SyntheticMessagesConfig, split: str):
        from datasets import Dataset

        rng = np.random.default_rng(config.seed + (0 if split == "train" else 7919))

        def sentence() -> str:
            return " ".join(f"w{int(i)}" for i in rng.integers(0, 5000, size=config.words_per_message))

        prompts, chosen, rejected = [], [], []
        for _ in range(config.num_samples):
            prompts.append([{"role": "user", "content": sentence()}])
            chosen.append([{"role": "assistant", "content": sentence()}])
            rejected.append([{"role": "assistant", "content": sentence()}])
        return Dataset.from_dict({"prompt": prompts, "chosen": chosen, "rejected": rejected})
