"""Contrastive training batches: pre-tokenised, pre-batched parquet data and a synthetic stand-in.

On-disk format (projects/arctic_embed/src/arctic_embed/core/pretokenized_batch_loader.py:52-406): a root directory
with one sub-directory ``batch_XXXXXXXX`` per global batch holding ``queries.parquet`` (``BATCH_QUERY_ID``,
``QUERY_TOKEN_ID_LIST``), ``documents.parquet`` (``BATCH_DOCUMENT_ID``, ``DOCUMENT_TOKEN_ID_LIST``) and
``relations.parquet`` (``BATCH_QUERY_ID``, ``BATCH_DOCUMENT_ID``, ``RELEVANCE``).  Every rank reads the same batch,
keeps a contiguous slice of the queries and of the documents (optionally ``split_factor`` sub-batches), while the
relevance matrix stays *global* (sparse COO) because the loss is taken over the gathered embeddings.
A one-thread read-ahead overlaps parquet decoding with the training step.
"""

from __future__ import annotations

import math
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass
from pathlib import Path
from typing import Any
from typing import Dict
from typing import Iterator
from typing import List
from typing import Optional
from typing import Sequence

import numpy as np
import torch
from pydantic import Field
from torch import Tensor

from ..config.data import DataConfig
from ..data.factory import DataFactory


@dataclass
class ContrastiveLearningBatch:
    query_tokens: Tensor
    query_attention_mask: Tensor
    document_tokens: Tensor
    document_attention_mask: Tensor
    relevance_labels: Tensor  # sparse COO [global queries, global documents]

    def to_device(self, device) -> "ContrastiveLearningBatch":
        return ContrastiveLearningBatch(*(t.to(device, non_blocking=True) for t in (
            self.query_tokens, self.query_attention_mask, self.document_tokens, self.document_attention_mask,
            self.relevance_labels)))


def pad_token_lists(rows: Sequence[Sequence[int]], pad_id: int, max_len: Optional[int], left_pad: bool = False):
    n = max((len(r) for r in rows), default=1)
    if max_len:
        n = min(n, max_len)
    ids = torch.full((len(rows), n), pad_id, dtype=torch.long)
    mask = torch.zeros((len(rows), n), dtype=torch.long)
    for i, r in enumerate(rows):
        r = list(r)[:n]
        if left_pad:
            ids[i, n - len(r):] = torch.as_tensor(r, dtype=torch.long)
            mask[i, n - len(r):] = 1
        else:
            ids[i, : len(r)] = torch.as_tensor(r, dtype=torch.long)
            mask[i, : len(r)] = 1
    return ids, mask


def shard_rows(n: int, rank: int, world: int) -> slice:
    per = n // world
    return slice(rank * per, (rank + 1) * per)


def slice_sparse_coo_tensor(t: Tensor, rows: slice, cols: slice) -> Tensor:
    """Sub-matrix of a 2-D sparse COO tensor (indices re-based), staying sparse."""
    t = t.coalesce()
    idx, val = t.indices(), t.values()
    r0, r1 = rows.start or 0, rows.stop if rows.stop is not None else t.size(0)
    c0, c1 = cols.start or 0, cols.stop if cols.stop is not None else t.size(1)
    keep = (idx[0] >= r0) & (idx[0] < r1) & (idx[1] >= c0) & (idx[1] < c1)
    new_idx = idx[:, keep] - torch.tensor([[r0], [c0]], device=idx.device)
    return torch.sparse_coo_tensor(new_idx, val[keep], (r1 - r0, c1 - c0))


def read_batch_dir(path: Path) -> Dict[str, Any]:
    import pyarrow.parquet as pq

    q = pq.read_table(path / "queries.parquet").to_pydict()
    d = pq.read_table(path / "documents.parquet").to_pydict()
    r = pq.read_table(path / "relations.parquet").to_pydict()
    q_order = np.argsort(q["BATCH_QUERY_ID"])
    d_order = np.argsort(d["BATCH_DOCUMENT_ID"])
    q_pos = {q["BATCH_QUERY_ID"][i]: n for n, i in enumerate(q_order)}
    d_pos = {d["BATCH_DOCUMENT_ID"][i]: n for n, i in enumerate(d_order)}
    rel_idx = torch.tensor([[q_pos[a] for a in r["BATCH_QUERY_ID"]], [d_pos[b] for b in r["BATCH_DOCUMENT_ID"]]],
                           dtype=torch.long)
    return {
        "queries": [q["QUERY_TOKEN_ID_LIST"][i] for i in q_order],
        "documents": [d["DOCUMENT_TOKEN_ID_LIST"][i] for i in d_order],
        "relations": torch.sparse_coo_tensor(rel_idx, torch.tensor(r["RELEVANCE"], dtype=torch.long),
                                             (len(q_order), len(d_order))),
    }


class PretokenizedBatchLoader:
    """Iterates the ``batch_*`` directories of one dataset, yielding this rank's :class:`ContrastiveLearningBatch`."""

    def __init__(self, root: Path, rank: int, world: int, pad_id: int = 0, max_query_len: Optional[int] = None,
                 max_doc_len: Optional[int] = None, split_factor: int = 1, left_pad: bool = False) -> None:
        self.root, self.rank, self.world = Path(root), rank, world
        self.pad_id, self.max_q, self.max_d, self.split, self.left_pad = pad_id, max_query_len, max_doc_len, split_factor, left_pad
        self.dirs = sorted(p for p in self.root.iterdir() if p.is_dir() and p.name.startswith("batch_"))
        if not self.dirs:
            raise FileNotFoundError(f"no batch_* directories under {self.root}")

    def __len__(self) -> int:
        return len(self.dirs) * self.split

    def _make(self, raw: Dict[str, Any], part: int) -> ContrastiveLearningBatch:
        nq, nd = len(raw["queries"]), len(raw["documents"])
        pq_, pd_ = nq // self.split, nd // self.split
        qs = slice(part * pq_, (part + 1) * pq_)
        ds = slice(part * pd_, (part + 1) * pd_)
        rel = slice_sparse_coo_tensor(raw["relations"], qs, ds) if self.split > 1 else raw["relations"]
        queries, docs = raw["queries"][qs], raw["documents"][ds]
        mq, md = shard_rows(len(queries), self.rank, self.world), shard_rows(len(docs), self.rank, self.world)
        q_ids, q_mask = pad_token_lists(queries[mq], self.pad_id, self.max_q, self.left_pad)
        d_ids, d_mask = pad_token_lists(docs[md], self.pad_id, self.max_d, self.left_pad)
        # rows that do not divide evenly over the ranks are dropped from the labels as well
        used_q, used_d = (len(queries) // self.world) * self.world, (len(docs) // self.world) * self.world
        rel = slice_sparse_coo_tensor(rel, slice(0, used_q), slice(0, used_d))
        return ContrastiveLearningBatch(q_ids, q_mask, d_ids, d_mask, rel)

    def __iter__(self) -> Iterator[ContrastiveLearningBatch]:
        with ThreadPoolExecutor(max_workers=1) as pool:
            nxt = pool.submit(read_batch_dir, self.dirs[0])
            for i in range(len(self.dirs)):
                raw = nxt.result()
                if i + 1 < len(self.dirs):
                    nxt = pool.submit(read_batch_dir, self.dirs[i + 1])
                for part in range(self.split):
                    yield self._make(raw, part)


class SyntheticContrastiveLoader:
    """Random token batches whose positives are a noisy copy of the query (so the loss can actually go down)."""

    def __init__(self, num_batches: int, global_queries: int, docs_per_query: int, seq_len: int, vocab: int, rank: int,
                 world: int, seed: int = 0) -> None:
        self.n, self.gq, self.dpq, self.seq, self.vocab, self.rank, self.world, self.seed = (
            num_batches, global_queries, docs_per_query, seq_len, vocab, rank, world, seed)

    def __len__(self) -> int:
        return self.n

    def __iter__(self) -> Iterator[ContrastiveLearningBatch]:
        g = torch.Generator().manual_seed(self.seed)
        for _ in range(self.n):
            q = torch.randint(8, self.vocab, (self.gq, self.seq), generator=g)
            docs = q.repeat_interleave(self.dpq, dim=0).clone()
            noise = torch.rand(docs.shape, generator=g) < 0.1
            docs[noise] = torch.randint(8, self.vocab, (int(noise.sum()),), generator=g)
            rows = torch.arange(self.gq).repeat_interleave(self.dpq)
            cols = torch.arange(self.gq * self.dpq)
            vals = torch.where(cols % self.dpq == 0, 1, -1)
            rel = torch.sparse_coo_tensor(torch.stack([rows, cols]), vals, (self.gq, self.gq * self.dpq))
            mq, md = shard_rows(self.gq, self.rank, self.world), shard_rows(self.gq * self.dpq, self.rank, self.world)
            yield ContrastiveLearningBatch(q[mq], torch.ones_like(q[mq]), docs[md], torch.ones_like(docs[md]), rel)


class ContrastivePretokenizedDataConfig(DataConfig):
    sources: List[Any] = Field(default_factory=list)
    filesystem: str = "local"
    root_directory: str = ""
    """ Directory with ``batch_*`` sub-directories (train). """
    eval_root_directories: List[str] = Field(default_factory=list)
    max_seq_length_query: Optional[int] = None
    max_seq_length_doc: Optional[int] = None
    pad_value: int = 0
    left_pad: bool = False
    split_factor: int = 1
    synthetic_batches: int = 0
    """ When > 0, ignore ``root_directory`` and generate this many synthetic batches. """
    synthetic_global_queries: int = 16
    synthetic_docs_per_query: int = 2
    synthetic_seq_len: int = 16
    synthetic_vocab: int = 1024


class ContrastivePretokenizedDataFactory(DataFactory):
    name = "contrastive_pretokenized"
    config: ContrastivePretokenizedDataConfig

    def __call__(self):
        c = self.config
        if c.synthetic_batches > 0:
            train = SyntheticContrastiveLoader(c.synthetic_batches, c.synthetic_global_queries, c.synthetic_docs_per_query,
                                               c.synthetic_seq_len, c.synthetic_vocab, self.global_rank, self.world_size, c.seed)
        else:
            train = PretokenizedBatchLoader(Path(c.root_directory), self.global_rank, self.world_size, c.pad_value,
                                            c.max_seq_length_query, c.max_seq_length_doc, c.split_factor, c.left_pad)
        evals = {Path(d).name: PretokenizedBatchLoader(Path(d), self.global_rank, self.world_size, c.pad_value,
                                                        c.max_seq_length_query, c.max_seq_length_doc, 1, c.left_pad)
                 for d in c.eval_root_directories}
        return train, (evals or None)

    def load(self, data_sources):
        raise NotImplementedError("pre-tokenised contrastive data is read batch by batch, not through data sources")

    def process(self, dataset):
        return dataset

    def split_data(self, training_data):
        return training_data, None

    def create_dataloader(self, dataset):
        return dataset
