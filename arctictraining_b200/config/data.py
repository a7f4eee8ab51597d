# SPDX-License-Identifier: Apache-2.0
"""``data:`` section and the per-source configs.  Parity: arctic_training/config/data.py:45-208."""

from __future__ import annotations

from pathlib import Path
from typing import TYPE_CHECKING
from typing import Any
from typing import Dict
from typing import List
from typing import Literal
from typing import Optional
from typing import Tuple
from typing import Type
from typing import Union

from pydantic import ValidationInfo
from pydantic import field_validator
from pydantic import model_validator
from typing_extensions import Self

from ..exceptions import RegistryError
from ..registry import _get_class_attr_type_hints
from ..registry import get_registered_data_factory
from ..registry import get_registered_data_source
from .base import BaseConfig
from .utils import HumanInt

if TYPE_CHECKING:
    from ..data.factory import DataFactory
    from ..data.source import DataSource


class DataSourceConfig(BaseConfig):
    """Fields common to every data source."""

    type: str = ""
    """ Data source type; a bare dataset name falls back to the factory's default source, then ``huggingface``. """

    split: str = ""
    """ Split to load; filled with ``train`` or ``eval`` when empty. """

    sample_ratio: Optional[float] = None
    """ Fraction of the examples to sample at random. """

    sample_count: Optional[int] = None
    """ Number of examples to sample at random. """

    sample_seed: int = 42
    """ Seed of the sampling above. """

    process: bool = True
    """ Run the data factory's ``process`` (tokenisation) on this source. """

    @property
    def data_source(self) -> Type["DataSource"]:
        return get_registered_data_source(self.type)

    @model_validator(mode="after")
    def _ratio_xor_count(self) -> Self:
        assert self.sample_ratio is None or self.sample_count is None, (
            "sample_ratio and sample_count cannot both be set."
        )
        return self


def _source_config_cls(source_type: str) -> type:
    return _get_class_attr_type_hints(get_registered_data_source(source_type), "config")[0]


class DataConfig(BaseConfig):
    type: str = ""
    """ Data factory type. Defaults to the first ``data_factory`` hint of the trainer. """

    sources: List[DataSourceConfig]
    """ Training data sources. """

    eval_sources: List[DataSourceConfig] = []
    """ Evaluation data sources. """

    train_eval_split: Tuple[float, float] = (1.0, 0.0)
    """ Fractions of the training data used for training and evaluation. """

    max_length: HumanInt = 8192
    """ Maximum length of the input sequence. """

    num_proc: int = 16
    """ Worker processes for tokenisation. """

    dl_num_workers: int = 2
    """ DataLoader workers per GPU. """

    seed: int = 42
    """ Seed of shuffling and sampling. """

    use_data_cache: Optional[bool] = None
    """ Deprecated (the cache is always used). """

    cache_processed_data: Optional[bool] = None
    """ Deprecated, see ``use_data_cache``. """

    cache_dir: Path = Path("/tmp/")
    """ Directory of the processed-data cache. """

    cache_fs_type: Literal["auto", "local", "shared"] = "auto"
    """ ``local``: local rank 0 of every node builds the cache; ``shared``: global rank 0 only. """

    fail_on_missing_cache: bool = False
    """ Raise instead of building a missing cache. """

    @property
    def factory(self) -> Type["DataFactory"]:
        return get_registered_data_factory(self.type)

    @field_validator("use_data_cache", "cache_processed_data", mode="after")
    @classmethod
    def _deprecated_cache_flags(cls, v: Optional[bool]) -> Optional[bool]:
        if v is not None:
            from ..logging import logger

            logger.warning("'use_data_cache' and 'cache_processed_data' are deprecated: the cache is always used.")
        return v

    @field_validator("cache_dir", mode="after")
    @classmethod
    def _absolute_cache_dir(cls, v: Path) -> Path:
        return v.resolve()

    @field_validator("sources", "eval_sources", mode="before")
    @classmethod
    def _build_source_configs(
        cls, v: List[Union[str, Dict[str, Any], DataSourceConfig]], info: ValidationInfo
    ) -> List[DataSourceConfig]:
        default_split = "train" if info.field_name == "sources" else "eval"
        factory_cls = get_registered_data_factory(info.data.get("type", ""))
        default_src = getattr(factory_cls, "default_source_cls", None)
        fallback = default_src.name if default_src is not None else "huggingface"
        out: List[DataSourceConfig] = []
        for item in v:
            if isinstance(item, str):
                base = item.split(":")[0]
                try:
                    get_registered_data_source(name=base)
                    src_type = base
                except RegistryError:
                    src_type = fallback
                out.append(_source_config_cls(src_type)(type=src_type, name_or_path=item, split=default_split))
            elif isinstance(item, dict):
                item = dict(item)
                item.setdefault("type", fallback)
                item.setdefault("split", default_split)
                out.append(_source_config_cls(item["type"])(**item))
            else:
                out.append(item)
        return out

    @model_validator(mode="after")
    def _finalise(self) -> Self:
        self.cache_dir.mkdir(parents=True, exist_ok=True)
        if self.eval_sources:
            assert self.train_eval_split[0] == 1.0, "train_eval_split should be (1.0, 0.0) when eval_sources is given."
        if self.train_eval_split[1] > 0.0:
            assert not self.eval_sources, "Give either an evaluation split or evaluation sources, not both."
        assert abs(sum(self.train_eval_split) - 1.0) < 1e-9, "train_eval_split should sum to 1.0."
        if self.cache_fs_type == "auto":
            from ..data.utils import is_local_fs

            object.__setattr__(self, "cache_fs_type", "local" if is_local_fs(self.cache_dir) else "shared")
        return self
