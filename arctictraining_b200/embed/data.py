# SPDX-License-Identifier: Apache-2.0
"""Contrastive training batches: pre-tokenised, pre-batched parquet data and a synthetic stand-in.

On-disk format (projects/arctic_embed/src/arctic_embed/core/pretokenized_batch_loader.py:52-406): a root directory
with one sub-directory ``batch_XXXXXXXX`` per global batch holding ``queries.parquet`` (``BATCH_QUERY_ID``,
``QUERY_TOKEN_ID_LIST``), ``documents.parquet`` (``BATCH_DOCUMENT_ID``, ``DOCUMENT_TOKEN_ID_LIST``) and
``relations.parquet`` (``BATCH_QUERY_ID``, ``BATCH_DOCUMENT_ID``, ``RELEVANCE``).  Every rank reads the same batch,
keeps a contiguous slice of the queries and of the documents (optionally ``split_factor`` sub-batches), while the
relevance matrix stays *global* (sparse COO) because the loss is taken over the gathered embeddings.
The root may live on any ``fsspec`` file system (local disk, S3, GCS, in-memory); a read-ahead pool overlaps fetching
and parquet decoding with the training step, and padding is one vectorised scatter per column.
"""

from __future__ import annotations

from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass
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


def open_filesystem(protocol: str = "local", **options):
    """An ``fsspec`` file system by protocol name (``local``, ``s3``, ``gs``, ``memory`` ...).  Object stores need their
    ``fsspec`` driver installed; the error of a missing one names it."""
    import fsspec

    return fsspec.filesystem("file" if protocol == "local" else protocol, **options)


def collate_token_column(column, pad_id: int, max_len: Optional[int], left_pad: bool = False):
    """Pad an arrow list column of token ids into ``(ids [n, L], mask [n, L])`` without a Python loop over rows:
    the flat value buffer is scattered with one fancy-index assignment."""
    arr = column.combine_chunks() if hasattr(column, "combine_chunks") else column
    offsets = arr.offsets.to_numpy().astype(np.int64)
    flat = arr.values.to_numpy(zero_copy_only=False).astype(np.int64, copy=False)
    lens = np.diff(offsets)
    n = len(lens)
    L = int(lens.max()) if n else 1
    if max_len:
        L = min(L, int(max_len))
    kept = np.minimum(lens, L)
    ids = np.full((n, max(L, 1)), pad_id, dtype=np.int64)
    col = np.arange(max(L, 1))[None, :]
    if left_pad:
        mask = col >= (L - kept)[:, None]
        src = offsets[:-1, None] + (col - (L - kept)[:, None])
    else:
        mask = col < kept[:, None]
        src = offsets[:-1, None] + col
    ids[mask] = flat[src[mask]]
    return torch.from_numpy(ids), torch.from_numpy(mask.astype(np.int64))


def read_batch_dir(path, filesystem=None) -> Dict[str, Any]:
    """One ``batch_*`` directory -> un-padded arrow token columns in id order + the sparse relevance matrix.  The three
    parquet files are fetched concurrently (on an object store the round trips dominate)."""
    import pyarrow.parquet as pq

    fs = filesystem or open_filesystem("local")
    base = str(path).rstrip("/")
    names = ("queries.parquet", "documents.parquet", "relations.parquet")
    with ThreadPoolExecutor(max_workers=3) as pool:
        q, d, r = pool.map(lambda n: pq.read_table(f"{base}/{n}", filesystem=fs), names)
    qids = q.column("BATCH_QUERY_ID").to_numpy()
    dids = d.column("BATCH_DOCUMENT_ID").to_numpy()
    if len(np.unique(qids)) != len(qids) or len(np.unique(dids)) != len(dids):
        raise ValueError(f"{base}: query / document ids must be unique inside a batch")
    q_order, d_order = np.argsort(qids, kind="stable"), np.argsort(dids, kind="stable")
    # position of every id after sorting: searchsorted on the sorted ids is the id -> row map
    rq = np.searchsorted(qids[q_order], r.column("BATCH_QUERY_ID").to_numpy())
    rd = np.searchsorted(dids[d_order], r.column("BATCH_DOCUMENT_ID").to_numpy())
    rel = torch.sparse_coo_tensor(torch.from_numpy(np.vstack([rq, rd]).astype(np.int64)),
                                  torch.from_numpy(r.column("RELEVANCE").to_numpy().astype(np.int64)),
                                  (len(qids), len(dids))).coalesce()
    return {
        "queries": q.column("QUERY_TOKEN_ID_LIST").take(q_order),
        "documents": d.column("DOCUMENT_TOKEN_ID_LIST").take(d_order),
        "relations": rel,
    }


def read_dataset_metadata(root: str, filesystem) -> Any:
    """``metadata.json`` written by the pre-tokeniser one or two levels above the batch directories, if present."""
    import json
    import posixpath

    parent = posixpath.dirname(str(root).rstrip("/"))
    for cand in (parent, posixpath.dirname(parent)):
        path = posixpath.join(cand, "metadata.json")
        if cand and filesystem.exists(path):
            return json.loads(filesystem.read_text(path))
    return None


class PretokenizedBatchLoader:
    """Iterates the ``batch_*`` directories of one dataset on any ``fsspec`` file system, yielding this rank's
    :class:`ContrastiveLearningBatch`.  ``read_ahead`` directories are fetched and decoded by background threads while
    the training step runs; with ``device`` set, each batch is copied there (pinned, non-blocking) one step early."""

    def __init__(self, root, rank: int, world: int, pad_id: int = 0, max_query_len: Optional[int] = None,
                 max_doc_len: Optional[int] = None, split_factor: int = 1, left_pad: bool = False, filesystem=None,
                 read_ahead: int = 2, device=None) -> None:
        self.fs = filesystem or open_filesystem("local")
        self.root, self.rank, self.world = str(root).rstrip("/"), rank, world
        self.pad_id, self.max_q, self.max_d, self.split, self.left_pad = pad_id, max_query_len, max_doc_len, split_factor, left_pad
        self.read_ahead, self.device = max(1, read_ahead), device
        listed = self.fs.ls(self.root, detail=False)
        self.dirs = sorted(p for p in listed if str(p).rstrip("/").rsplit("/", 1)[-1].startswith("batch_"))
        if not self.dirs:
            raise FileNotFoundError(f"no batch_* directories under {self.root}")

    def __len__(self) -> int:
        return len(self.dirs) * self.split

    def _make(self, raw: Dict[str, Any], part: int) -> ContrastiveLearningBatch:
        nq, nd = len(raw["queries"]), len(raw["documents"])
        pq_, pd_ = nq // self.split, nd // self.split
        rel = slice_sparse_coo_tensor(raw["relations"], slice(part * pq_, (part + 1) * pq_),
                                      slice(part * pd_, (part + 1) * pd_)) if self.split > 1 else raw["relations"]
        mq, md = shard_rows(pq_, self.rank, self.world), shard_rows(pd_, self.rank, self.world)
        queries = raw["queries"].slice(part * pq_ + mq.start, mq.stop - mq.start)
        docs = raw["documents"].slice(part * pd_ + md.start, md.stop - md.start)
        q_ids, q_mask = collate_token_column(queries, self.pad_id, self.max_q, self.left_pad)
        d_ids, d_mask = collate_token_column(docs, self.pad_id, self.max_d, self.left_pad)
        # rows that do not divide evenly over the ranks are dropped from the labels as well
        used_q, used_d = (pq_ // self.world) * self.world, (pd_ // self.world) * self.world
        rel = slice_sparse_coo_tensor(rel, slice(0, used_q), slice(0, used_d))
        return ContrastiveLearningBatch(q_ids, q_mask, d_ids, d_mask, rel)

    def _load(self, path) -> List[ContrastiveLearningBatch]:
        raw = read_batch_dir(path, self.fs)
        return [self._make(raw, part) for part in range(self.split)]

    def _stage(self, batch: ContrastiveLearningBatch) -> ContrastiveLearningBatch:
        if self.device is None:
            return batch
        pinned = ContrastiveLearningBatch(*(t.pin_memory() if not t.is_sparse and torch.cuda.is_available() else t
                                            for t in (batch.query_tokens, batch.query_attention_mask, batch.document_tokens,
                                                      batch.document_attention_mask, batch.relevance_labels)))
        return pinned.to_device(self.device)

    def __iter__(self) -> Iterator[ContrastiveLearningBatch]:
        meta = read_dataset_metadata(self.root, self.fs)
        from ..logging import logger

        logger.info(f"iterating {self.root} ({len(self.dirs)} batch directories; tokenisation: {meta or 'no metadata'})")
        with ThreadPoolExecutor(max_workers=self.read_ahead) as pool:
            pending = [pool.submit(self._load, p) for p in self.dirs[: self.read_ahead]]
            nxt = self.read_ahead
            staged = None
            while pending:
                parts = pending.pop(0).result()
                if nxt < len(self.dirs):
                    pending.append(pool.submit(self._load, self.dirs[nxt]))
                    nxt += 1
                for b in parts:  # copy batch i+1 to the device before handing out batch i
                    b = self._stage(b)
                    if staged is not None:
                        yield staged
                    staged = b
            if staged is not None:
                yield staged


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
    """ ``fsspec`` protocol of the data: ``local``, ``s3``, ``gs``, ``memory`` ... """
    filesystem_options: Dict[str, Any] = Field(default_factory=dict)
    """ Keyword arguments of the file system (credentials, endpoint, ...). """
    read_ahead: int = 2
    """ Batch directories fetched and decoded ahead of the training step. """
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
            fs = open_filesystem(c.filesystem, **c.filesystem_options)
            train = PretokenizedBatchLoader(c.root_directory, self.global_rank, self.world_size, c.pad_value,
                                            c.max_seq_length_query, c.max_seq_length_doc, c.split_factor, c.left_pad,
                                            filesystem=fs, read_ahead=c.read_ahead)
        evals = {}
        for d in c.eval_root_directories:
            fs = open_filesystem(c.filesystem, **c.filesystem_options)
            evals[d.rstrip("/").rsplit("/", 1)[-1]] = PretokenizedBatchLoader(
                d, self.global_rank, self.world_size, c.pad_value, c.max_seq_length_query, c.max_seq_length_doc, 1,
                c.left_pad, filesystem=fs, read_ahead=c.read_ahead)
        return train, (evals or None)

    def load(self, data_sources):
        raise NotImplementedError("pre-tokenised contrastive data is read batch by batch, not through data sources")

    def process(self, dataset):
        return dataset

    def split_data(self, training_data):
        return training_data, None

    def create_dataloader(self, dataset):
        return dataset
