# SPDX-License-Identifier: Apache-2.0
"""Snowflake data source: SQL query, whole table, or versioned Snowflake Dataset.

Behaviour parity: arctic_training/data/snowflake_source.py:33-233 (three mutually exclusive modes,
``snow://dataset/<name>/versions/<version>`` URIs, optional column renaming, row limit).  The Snowflake
client libraries are imported only when data is actually loaded.
"""

from __future__ import annotations

import re
from typing import Any
from typing import Dict
from typing import Optional

from pydantic import Field
from pydantic import model_validator
from typing_extensions import Self

from ..config.data import DataSourceConfig
from .source import DataSource

_DATASET_URI = re.compile(r"^snow://dataset/([^/]+)/versions/([^/]+)$")
_IDENT = r'(?:[A-Za-z_][A-Za-z0-9_$]*|"(?:[^"]|"")+")'
_OBJECT_NAME = re.compile(rf"^{_IDENT}(?:\.{_IDENT}){{0,2}}$")


def _require_snowflake() -> None:
    try:
        import snowflake.ml  # noqa: F401
    except ImportError as exc:
        raise ImportError("snowflake-ml-python is required for Snowflake data sources.") from exc


def get_default_snowflake_session() -> Any:
    """An active Snowpark session, or a new one from the environment / ``~/.snowflake`` configuration."""
    _require_snowflake()
    from snowflake.snowpark import Session

    try:
        return Session.builder.getOrCreate()
    except Exception:
        from snowflake.ml._internal.utils.connection_params import SnowflakeLoginOptions

        return Session.builder.configs(SnowflakeLoginOptions()).getOrCreate()


class SnowflakeSourceConfig(DataSourceConfig):
    sql: Optional[str] = None
    """ SQL query to run. """

    table_name: Optional[str] = None
    """ ``[[db.]schema.]table`` to read completely. """

    dataset_uri: Optional[str] = None
    """ ``snow://dataset/<[[db.]schema.]name>/versions/<version>``. """

    column_mapping: Dict[str, str] = Field(default_factory=dict)
    """ Source column -> target column renames. """

    limit: Optional[int] = None
    """ Maximum number of rows. """

    batch_size: int = 1024
    """ Batch size of the internal reader. """

    @model_validator(mode="after")
    def _exactly_one_mode(self) -> Self:
        if sum(x is not None for x in (self.sql, self.table_name, self.dataset_uri)) != 1:
            raise ValueError("Exactly one of 'sql', 'table_name', or 'dataset_uri' must be specified")
        if self.table_name:
            object.__setattr__(self, "sql", f"SELECT * FROM {self.table_name}")
        if self.dataset_uri:
            m = _DATASET_URI.match(self.dataset_uri)
            if not m:
                raise ValueError(
                    f"Invalid dataset_uri format: '{self.dataset_uri}'. "
                    "Expected format: 'snow://dataset/<dataset_name>/versions/<version_name>'"
                )
            if not _OBJECT_NAME.match(m.group(1)):
                raise ValueError(f"Invalid dataset_name format in URI: {m.group(1)!r}")
        return self


class SnowflakeDataSource(DataSource):
    name = "snowflake"
    config: SnowflakeSourceConfig

    session: Optional[Any] = None
    """ Snowpark session to use; a default one is created when ``None``. """

    def load(self, config: SnowflakeSourceConfig, split: str):
        _require_snowflake()
        session = self.session or get_default_snowflake_session()
        from snowflake.ml.data.data_connector import DataConnector

        if config.dataset_uri:
            from snowflake.ml.dataset import load_dataset

            m = _DATASET_URI.match(config.dataset_uri)
            assert m is not None
            connector = DataConnector.from_dataset(load_dataset(session, m.group(1), m.group(2)))
        else:
            connector = DataConnector.from_sql(config.sql, session=session)
        return connector.to_huggingface_dataset(streaming=False, limit=config.limit, batch_size=config.batch_size)

    def post_load_callback(self, dataset):
        if self.config.column_mapping:
            dataset = dataset.rename_columns(self.config.column_mapping)
        return dataset
