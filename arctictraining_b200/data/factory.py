# SPDX-License-Identifier: Apache-2.0
"""Data factory base class.  Parity: arctic_training/data/factory.py:50-239 — the main process (local
rank 0 on a node-local cache, global rank 0 on a shared one) builds the concatenated and shuffled
dataset, replicates it up to ``min_iterations``, publishes it atomically, everybody meets at a barrier,
reseeds and memory-maps the result; then train/eval split and ``DataLoader`` creation with a
``DistributedSampler`` over the whole world and ``drop_last=True``."""

from __future__ import annotations

from abc import ABC
from pathlib import Path
from typing import TYPE_CHECKING
from typing import Any
from typing import List
from typing import Optional
from typing import Tuple
from typing import Type

import torch
from torch.utils.data import DataLoader
from torch.utils.data import DistributedSampler

from ..callback.mixin import CallbackMixin
from ..callback.mixin import callback_wrapper
from ..comm import dist as cdist
from ..config.data import DataConfig
from ..config.data import DataSourceConfig
from ..logging import logger
from ..registry import RegistryMeta
from ..registry import _validate_class_attribute_set
from ..registry import _validate_class_attribute_type
from ..registry import _validate_class_method
from .utils import calculate_hash_from_args

if TYPE_CHECKING:
    from ..trainer.trainer import Trainer
    from .source import DataSource


class DataFactory(ABC, CallbackMixin, metaclass=RegistryMeta):
    name: str
    """ Name under which the factory is selected in a recipe (``data.type``). """

    config: DataConfig
    """ Config class of this factory. """

    default_source_cls: Optional[Type] = None

    @classmethod
    def _validate_subclass(cls) -> None:
        _validate_class_attribute_set(cls, "name")
        _validate_class_attribute_type(cls, "config", DataConfig)
        _validate_class_method(cls, "load", ["self", "data_sources"])
        _validate_class_method(cls, "process", ["self", "dataset"])
        _validate_class_method(cls, "split_data", ["self", "training_data"])
        _validate_class_method(cls, "create_dataloader", ["self", "dataset"])

    def __init__(self, trainer: "Trainer", config: Optional[DataConfig] = None) -> None:
        self._trainer = trainer
        self.config = config if config is not None else trainer.config.data

    # ------------------------------------------------------------------ orchestration
    def _get_data_sources(self, data_source_configs: List[DataSourceConfig]) -> List["DataSource"]:
        """One data-source object per configured source, bound to this factory."""
        return [c.data_source(data_factory=self, config=c) for c in data_source_configs]

    def _load_sources(self, cfgs: List[DataSourceConfig]):
        from datasets import concatenate_datasets
        from datasets import load_from_disk

        if not cfgs:
            return None
        sources = self._get_data_sources(cfgs)
        cache_path = self.cache_path(sources)
        if self.is_main_process_by_path and not cache_path.exists():
            if self.config.fail_on_missing_cache:
                raise FileNotFoundError(f"Cache path {cache_path.as_posix()} does not exist.")
            dataset = self.load(sources)
            tc = self.trainer.config
            if tc.min_iterations > 0:
                need = tc.min_iterations * tc.micro_batch_size * tc.gradient_accumulation_steps * self.world_size
                if need > len(dataset):
                    dataset = concatenate_datasets([dataset] * (need // len(dataset) + 1)).select(range(need))
            if len(dataset) < self.world_size:
                raise ValueError(
                    f"Dataset size ({len(dataset)}) is less than the data parallel size ({self.world_size}); "
                    "set `min_iterations` to replicate the data for development runs."
                )
            tmp = cache_path.with_suffix(".incomplete")
            dataset.save_to_disk(tmp.as_posix())
            tmp.rename(cache_path)
        try:
            cdist.barrier()
        except (RuntimeError, KeyboardInterrupt):
            # the main process most likely failed while preparing the data: leave quietly
            raise SystemExit(1)
        self.trainer._set_seeds(self.trainer.config.seed)
        logger.info(f"Loading dataset from cache path {cache_path.as_posix()}")
        return load_from_disk(cache_path.as_posix())

    def __call__(self) -> Tuple[Any, Optional[Any]]:
        train = self._load_sources(self.config.sources)
        evald = self._load_sources(self.config.eval_sources)
        if self.config.train_eval_split[1] > 0.0:
            train, evald = self.split_data(train)
        train_dl = self.create_dataloader(train)
        eval_dl = self.create_dataloader(evald) if evald is not None else None
        return train_dl, eval_dl

    # ------------------------------------------------------------------ accessors
    @property
    def trainer(self) -> "Trainer":
        return self._trainer

    @property
    def tokenizer(self):
        return self.trainer.tokenizer

    @property
    def micro_batch_size(self) -> int:
        return self.trainer.config.micro_batch_size

    @property
    def global_rank(self) -> int:
        return self.config.global_rank

    @property
    def local_rank(self) -> int:
        return self.config.local_rank

    @property
    def world_size(self) -> int:
        return self.config.world_size

    @property
    def is_main_process_by_path(self) -> bool:
        return self.local_rank == 0 if self.config.cache_fs_type == "local" else self.global_rank == 0

    def cache_path(self, sources: List["DataSource"]) -> Path:
        return self.config.cache_dir / calculate_hash_from_args(*[s.cache_path_args for s in sources])

    # ------------------------------------------------------------------ overridable steps
    @callback_wrapper("load")
    def load(self, data_sources: List["DataSource"]):
        from datasets import concatenate_datasets

        return concatenate_datasets([s() for s in data_sources]).shuffle(seed=self.config.seed)

    @callback_wrapper("process")
    def process(self, dataset):
        raise NotImplementedError("process must be implemented by the DataFactory subclass")

    @callback_wrapper("split")
    def split_data(self, training_data):
        parts = training_data.train_test_split(test_size=self.config.train_eval_split[1], seed=self.config.seed)
        return parts["train"], parts["test"]

    def collate_fn(self):
        return None

    @callback_wrapper("create_dataloader")
    def create_dataloader(self, dataset) -> DataLoader:
        workers = self.config.dl_num_workers
        return DataLoader(
            dataset,
            batch_size=self.micro_batch_size,
            sampler=DistributedSampler(dataset, num_replicas=self.world_size, rank=self.global_rank),
            num_workers=workers,
            persistent_workers=workers > 0,
            collate_fn=self.collate_fn(),
            pin_memory=torch.cuda.is_available(),
            drop_last=True,
        )
