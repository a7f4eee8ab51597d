# SPDX-License-Identifier: Apache-2.0
"""Teacher / mining embedders and small helpers of the data-preparation jobs.

Parity: projects/arctic_embed/src/arctic_embed/data_processing/teacher_models.py:40-95 (embedder interface and the
Arctic-Embed 2.0 large teacher), utils.py:44-148 (pooling, normalisation, embedding parquet I/O, config-file CLI).
"""

from __future__ import annotations

import sys
from abc import ABC
from abc import abstractmethod
from typing import Any
from typing import Callable
from typing import Optional
from typing import Sequence
from typing import Type

import numpy as np
import torch
from pydantic import BaseModel

from ..model import pool


class Embedder(ABC):
    """Maps texts to unit-norm vectors; queries and documents may use different prefixes."""

    @abstractmethod
    def to_device(self, device) -> None: ...

    @abstractmethod
    def embed_batch(self, texts: Sequence[str], is_query: bool, **kwargs: Any) -> np.ndarray: ...

    def embed_all(self, texts: Sequence[str], is_query: bool, batch_size: int = 256, **kwargs: Any) -> np.ndarray:
        """All texts, longest first (batches of similar length waste the least padding), returned in input order."""
        order = np.argsort([-len(t) for t in texts], kind="stable")
        out: Optional[np.ndarray] = None
        for s in range(0, len(texts), batch_size):
            sel = order[s : s + batch_size]
            emb = self.embed_batch([texts[i] for i in sel], is_query, **kwargs)
            if out is None:
                out = np.empty((len(texts), emb.shape[1]), dtype=emb.dtype)
            out[sel] = emb
        return out if out is not None else np.empty((0, 0), dtype=np.float32)


class HFEmbedder(Embedder):
    """Any Hugging Face encoder with a pooling rule (``first_token``, ``last_token``, ``mean``) and text prefixes.
    ``HFEmbedder.arctic_embed_2_large()`` gives the teacher the reference ships (CLS pooling, ``query: `` prefix)."""

    def __init__(self, model_name_or_path: str, pooling: str = "first_token", query_prefix: str = "", document_prefix: str = "",
                 max_seq_len: int = 8192, dtype: torch.dtype = torch.bfloat16, model=None, tokenizer=None) -> None:
        if model is None or tokenizer is None:
            from transformers import AutoModel
            from transformers import AutoTokenizer

            tokenizer = tokenizer or AutoTokenizer.from_pretrained(model_name_or_path)
            model = model or AutoModel.from_pretrained(model_name_or_path, torch_dtype=dtype, add_pooling_layer=False)
        self.model, self.tokenizer = model.eval(), tokenizer
        self.pooling, self.qp, self.dp, self.max_seq_len = pooling, query_prefix, document_prefix, max_seq_len
        self.device = torch.device("cpu")

    @classmethod
    def arctic_embed_2_large(cls, max_seq_len: int = 8192) -> "HFEmbedder":
        return cls("Snowflake/snowflake-arctic-embed-l-v2.0", "first_token", "query: ", "", max_seq_len)

    def to_device(self, device) -> None:
        self.device = torch.device(device)
        self.model.to(self.device)

    @torch.inference_mode()
    def embed_batch(self, texts: Sequence[str], is_query: bool, max_seq_len: Optional[int] = None, **kwargs: Any) -> np.ndarray:
        prefix = self.qp if is_query else self.dp
        enc = self.tokenizer([prefix + t for t in texts], padding=True, truncation=True,
                             max_length=max_seq_len or self.max_seq_len, return_tensors="pt")
        enc = {k: v.to(self.device) for k, v in enc.items()}
        hidden = self.model(**enc)[0]
        emb = torch.nn.functional.normalize(pool(hidden, enc["attention_mask"], self.pooling).float(), dim=-1)
        return emb.cpu().numpy()


def normalize_embeddings(matrix: np.ndarray) -> np.ndarray:
    """Row-wise L2 normalisation in place (returns the same array)."""
    norms = np.linalg.norm(matrix, axis=1, keepdims=True)
    np.divide(matrix, np.maximum(norms, 1e-12), out=matrix)
    return matrix


def write_embeddings(location: str, ids: Sequence, matrix: np.ndarray, id_col: str = "ID", vec_col: str = "VECTOR") -> None:
    import pyarrow as pa
    import pyarrow.parquet as pq

    from .parquet_store import filesystem_for

    import posixpath

    fs, path = filesystem_for(location)
    if posixpath.dirname(path):
        fs.makedirs(posixpath.dirname(path), exist_ok=True)
    flat = pa.array(np.ascontiguousarray(matrix).reshape(-1))
    vecs = pa.FixedSizeListArray.from_arrays(flat, matrix.shape[1])
    pq.write_table(pa.table({id_col: pa.array(list(ids)), vec_col: vecs}), path, filesystem=fs)


def read_embeddings(location: str, id_col: str = "ID", vec_col: str = "VECTOR"):
    """``(ids, matrix [n, d])`` from one parquet file or a directory of them."""
    from .parquet_store import ParquetCollection

    table = ParquetCollection.from_location(location).read_all([id_col, vec_col])
    col = table.column(vec_col).combine_chunks()
    dim = col.type.list_size if hasattr(col.type, "list_size") else len(col[0])
    flat = (col.flatten() if hasattr(col, "flatten") else col.values).to_numpy(zero_copy_only=False)
    return table.column(id_col).to_numpy(zero_copy_only=False), flat.reshape(-1, dim)


def run_config_file_cli(config_cls: Type[BaseModel], job: Callable[[Any], None], argv: Optional[Sequence[str]] = None) -> None:
    """``prog CONFIG.{json,yaml} [--shard I --num-shards N]``: validate the file as ``config_cls`` and run ``job``."""
    import argparse
    import json

    import yaml

    ap = argparse.ArgumentParser(description=(job.__doc__ or "").strip().split("\n")[0])
    ap.add_argument("config")
    ap.add_argument("--shard", type=int, default=None)
    ap.add_argument("--num-shards", type=int, default=None)
    args = ap.parse_args(list(argv) if argv is not None else sys.argv[1:])
    text = open(args.config).read()
    raw = json.loads(text) if args.config.endswith(".json") else yaml.safe_load(text)
    cfg = config_cls.model_validate(raw)
    if args.num_shards:
        cfg = cfg.split_to_shards(args.num_shards)[args.shard or 0]
    job(cfg)
