# SPDX-License-Identifier: Apache-2.0
"""Data source base class.  Parity: arctic_training/data/source.py:41-168 — per-source cache keyed by an
md5 of (factory config, source config, tokenizer config), optional random sub-sampling, tokenisation
by the owning factory, atomic ``.incomplete`` -> rename publication, memory-mapped reload."""

from __future__ import annotations

import random
from abc import ABC
from abc import abstractmethod
from functools import cached_property
from pathlib import Path
from typing import TYPE_CHECKING
from typing import Any
from typing import Dict
from typing import Tuple

from ..callback.mixin import CallbackMixin
from ..callback.mixin import callback_wrapper
from ..config.data import DataSourceConfig
from ..logging import logger
from ..registry import RegistryMeta
from ..registry import _validate_class_attribute_set
from ..registry import _validate_class_attribute_type
from ..registry import _validate_class_method
from .utils import calculate_hash_from_args

if TYPE_CHECKING:
    from .factory import DataFactory

_CACHE_IRRELEVANT = {"sources", "eval_sources", "cache_dir", "num_proc", "train_eval_split", "use_data_cache",
                     "cache_processed_data", "dl_num_workers", "cache_fs_type", "fail_on_missing_cache"}


class DataSource(ABC, CallbackMixin, metaclass=RegistryMeta):
    name: str
    """ Name under which the source is selected in a recipe. """

    config: DataSourceConfig
    """ Config class of this source. """

    @classmethod
    def _validate_subclass(cls) -> None:
        _validate_class_attribute_set(cls, "name")
        _validate_class_attribute_type(cls, "config", DataSourceConfig)
        _validate_class_method(cls, "load", ["self", "config", "split"])

    def __init__(self, data_factory: "DataFactory", config: DataSourceConfig) -> None:
        self._data_factory = data_factory
        self.config = config

    def __call__(self):
        from datasets import disable_caching
        from datasets import load_from_disk

        disable_caching()
        if self.cache_path.exists():
            logger.info(f"Loading data source from cache path {self.cache_path.as_posix()}")
            return load_from_disk(self.cache_path.as_posix())
        dataset = self.load(self.config, self.config.split)
        count = None
        if self.config.sample_ratio is not None:
            count = int(len(dataset) * self.config.sample_ratio)
        elif self.config.sample_count is not None:
            count = self.config.sample_count
        if count is not None:
            if count >= len(dataset):
                logger.warning(f"Requested {count} samples but {self.name} only has {len(dataset)}; using all.")
            else:
                rng = random.Random(self.config.sample_seed)
                dataset = dataset.select(rng.sample(range(len(dataset)), count))
        if len(dataset) < 1:
            raise ValueError(f"Empty dataset from load() for data source {self.name} split {self.config.split}")
        if self.config.process:
            dataset = self.data_factory.process(dataset)
            if len(dataset) < 1:
                raise ValueError(f"Empty dataset after process() for data source {self.name}")
        tmp = self.cache_path.with_suffix(".incomplete")
        dataset.save_to_disk(tmp.as_posix())
        tmp.rename(self.cache_path)
        return load_from_disk(self.cache_path.as_posix())

    @property
    def data_factory(self) -> "DataFactory":
        return self._data_factory

    @property
    def trainer(self):
        return self._data_factory.trainer

    @property
    def world_size(self) -> int:
        return self._data_factory.world_size

    @property
    def global_rank(self) -> int:
        return self._data_factory.global_rank

    @property
    def cache_path_args(self) -> Tuple[Dict[str, Any], ...]:
        return (
            self.data_factory.config.model_dump(exclude=_CACHE_IRRELEVANT, mode="json"),
            self.config.model_dump(mode="json"),
            self.trainer.config.tokenizer.model_dump(mode="json"),
        )

    @cached_property
    def cache_path(self) -> Path:
        return self.data_factory.config.cache_dir / calculate_hash_from_args(*self.cache_path_args)

    @callback_wrapper("load")
    @abstractmethod
    def load(self, config: DataSourceConfig, split: str):
        """Return a ``datasets.Dataset`` with the columns the owning data factory expects."""
        raise NotImplementedError
