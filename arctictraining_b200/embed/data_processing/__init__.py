# SPDX-License-Identifier: Apache-2.0
"""Offline data preparation for contrastive embedding training: parquet collections on any file system, dense
retrieval for hard-negative mining, teacher embedders, and the two pre-tokenise-and-batch jobs that write the
``batch_*`` layout the training loader streams.  Parity: projects/arctic_embed/src/arctic_embed/data_processing/."""

from .embedders import Embedder
from .embedders import HFEmbedder
from .embedders import run_config_file_cli
from .mining import combine_datasets
from .mining import mine_hard_negatives
from .mining import scramble_ids
from .parquet_store import ParquetCollection
from .parquet_store import filesystem_for
from .retrieval import dense_retrieval
from .tokenize_jobs import JobShard
from .tokenize_jobs import MinedDataJob
from .tokenize_jobs import PairsJob
from .tokenize_jobs import pretokenize_mined_data
from .tokenize_jobs import pretokenize_pairs
from .tokenize_jobs import shard_row_range
