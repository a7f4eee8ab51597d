# SPDX-License-Identifier: Apache-2.0
"""The two pre-tokenise-and-batch jobs.  Both write ``<out>/metadata.json`` and ``batch_XXXXXXXX/{queries,documents,
relations}.parquet`` with batch-local integer ids — the layout ``PretokenizedBatchLoader`` streams.

* :func:`pretokenize_pairs` — large-scale (query, document) pairs: every ``batch_size`` consecutive input rows form one
  batch, queries and documents are de-duplicated by id inside the batch, every pair is a positive.  A job can be cut
  into shards that own whole batches, so shards run in parallel and write disjoint directories.
* :func:`pretokenize_mined_data` — the output of hard-negative mining: per query one (or a few) sampled positives and
  the top negatives; with ``num_query_uses > 1`` every query appears in that many batches with disjoint negatives.

Parity: projects/arctic_embed/src/arctic_embed/data_processing/pretokenize.py:45-786.
"""

from __future__ import annotations

import json
import posixpath
from typing import Callable
from typing import List
from typing import Optional
from typing import Sequence
from typing import Tuple

import numpy as np
from pydantic import BaseModel
from pydantic import ConfigDict

from ...logging import logger
from .parquet_store import ParquetCollection
from .parquet_store import filesystem_for

TokenizeFn = Callable[[Sequence[str]], List[List[int]]]


class _Strict(BaseModel):
    model_config = ConfigDict(extra="forbid", validate_default=True, use_attribute_docstrings=True)


class JobShard(_Strict):
    shard_id: int = 0
    num_shards: int = 1


class _TokenizedOutput(_Strict):
    tokenizer_id: str
    """ Hugging Face hub id or local directory of the tokenizer. """
    query_prefix: str = ""
    document_prefix: str = ""
    max_seq_length: int = 1024
    pre_truncate_max_chars_per_token: int = 8
    """ Texts are cut to ``max_seq_length x`` this many characters before tokenising (bounds tokeniser time on very
    long inputs; 8 is safe for English). """
    out_query_id_col: str = "BATCH_QUERY_ID"
    out_document_id_col: str = "BATCH_DOCUMENT_ID"
    out_query_tokens_col: str = "QUERY_TOKEN_ID_LIST"
    out_document_tokens_col: str = "DOCUMENT_TOKEN_ID_LIST"
    out_relevance_col: str = "RELEVANCE"


class PairsJob(_TokenizedOutput):
    query_doc_pair_dir: str
    output_dir: str
    batch_size: int = 32_000
    pair_query_id_col: str = "QUERY_ID"
    pair_document_id_col: str = "DOCUMENT_ID"
    pair_query_text_col: str = "QUERY_TEXT"
    pair_document_text_col: str = "DOCUMENT_TEXT"
    shard_info: JobShard = JobShard()

    def split_to_shards(self, num_shards: int) -> List["PairsJob"]:
        if self.shard_info.num_shards > 1:
            raise ValueError("this job is already one shard of a larger job")
        return [self.model_copy(update={"shard_info": JobShard(shard_id=i, num_shards=num_shards)}) for i in range(num_shards)]


class MinedDataJob(_TokenizedOutput):
    query_loc: str
    document_loc: str
    labels_loc: str
    output_loc: str
    random_seed: int = 0
    queries_per_batch: int = 256
    num_query_uses: int = 1
    num_negatives_per_query_per_batch: int = 10
    max_pos_per_query: int = 1
    in_query_id_col: str = "QUERY_ID"
    in_document_id_col: str = "DOCUMENT_ID"
    in_query_text_col: str = "QUERY_TEXT"
    in_document_text_col: str = "DOCUMENT_TEXT"
    in_label_relation_col: str = "RELEVANCE"


def shard_row_range(num_rows: int, chunk_size: int, shard_id: int, num_shards: int) -> Tuple[int, int]:
    """Rows ``[start, stop)`` of a shard that owns whole chunks: chunks are dealt out as evenly as possible, earlier
    shards taking the extra ones; the last chunk may be partial."""
    if not 0 <= shard_id < num_shards:
        raise ValueError(f"shard {shard_id} of {num_shards}")
    chunks = -(-num_rows // chunk_size)
    base, extra = divmod(chunks, num_shards)
    first = shard_id * base + min(shard_id, extra)
    count = base + (1 if shard_id < extra else 0)
    return min(num_rows, first * chunk_size), min(num_rows, (first + count) * chunk_size)


def load_tokenizer(tokenizer_id: str) -> TokenizeFn:
    """A batch tokenise function without padding or truncation (the jobs truncate themselves)."""
    from tokenizers import Tokenizer
    import os

    path = os.path.join(tokenizer_id, "tokenizer.json")
    tok = Tokenizer.from_file(path) if os.path.exists(path) else Tokenizer.from_pretrained(tokenizer_id)
    tok.no_padding()
    tok.no_truncation()
    return lambda texts: [e.ids for e in tok.encode_batch(list(texts))]


def tokenize_to_arrow(tokenize: TokenizeFn, texts: Sequence[str], max_length: int, pre_truncate_max_chars_per_token: int,
                      chunk: int = 4096):
    """Arrow ``list<int32>`` of token ids, truncated to ``max_length``, tokenised ``chunk`` texts at a time."""
    import pyarrow as pa

    limit = max_length * pre_truncate_max_chars_per_token
    pieces = []
    for s in range(0, len(texts), chunk):
        ids = tokenize([t[:limit] for t in texts[s : s + chunk]])
        pieces.append(pa.array([row[:max_length] for row in ids], type=pa.list_(pa.int32())))
    return pa.chunked_array(pieces, type=pa.list_(pa.int32())) if pieces else pa.array([], type=pa.list_(pa.int32()))


def _write_metadata(fs, root: str, meta: dict) -> None:
    fs.makedirs(root, exist_ok=True)
    path = posixpath.join(root, "metadata.json")
    if fs.exists(path):  # shards of one job all try; the first wins
        return
    with fs.open(path, "w") as f:
        f.write(json.dumps(meta, indent=2))


def _write_batch(fs, root: str, index: int, tables: dict) -> None:
    import pyarrow.parquet as pq

    out = posixpath.join(root, f"batch_{index:08d}")
    fs.makedirs(out, exist_ok=True)
    for name, table in tables.items():
        pq.write_table(table, posixpath.join(out, name), filesystem=fs)


def _fill_missing_ids(ids: np.ndarray, texts: np.ndarray) -> np.ndarray:
    """Rows without an id get one derived from their text, so equal texts still de-duplicate."""
    import zlib

    ids = ids.astype(object)
    for i in np.flatnonzero([v is None or (isinstance(v, float) and np.isnan(v)) for v in ids]):
        ids[i] = f"__MISSING_ID__{zlib.crc32(str(texts[i]).encode()):08x}{len(str(texts[i]))}"
    return ids


def pretokenize_pairs(config: PairsJob, tokenize: Optional[TokenizeFn] = None) -> int:
    """Pre-tokenise and batch (query, document) pairs; returns the number of batches this shard wrote."""
    import pyarrow as pa

    c = config
    tokenize = tokenize or load_tokenizer(c.tokenizer_id)
    src = ParquetCollection.from_location(c.query_doc_pair_dir)
    start, stop = shard_row_range(src.num_rows, c.batch_size, c.shard_info.shard_id, c.shard_info.num_shards)
    fs, out_root = filesystem_for(c.output_dir)
    _write_metadata(fs, out_root, {"tokenizer_huggingface_id": c.tokenizer_id, "batch_size": c.batch_size,
                                   "max_seq_length": c.max_seq_length, "query_prefix": c.query_prefix,
                                   "document_prefix": c.document_prefix})
    cols = [c.pair_query_id_col, c.pair_document_id_col, c.pair_query_text_col, c.pair_document_text_col]
    first_batch = start // c.batch_size
    written = 0
    for i, table in enumerate(src.stream_chunks(c.batch_size, cols, (start, stop))):
        q_text = table[c.pair_query_text_col].to_numpy(zero_copy_only=False)
        d_text = table[c.pair_document_text_col].to_numpy(zero_copy_only=False)
        qid = _fill_missing_ids(table[c.pair_query_id_col].to_numpy(zero_copy_only=False), q_text).astype(str)
        did = _fill_missing_ids(table[c.pair_document_id_col].to_numpy(zero_copy_only=False), d_text).astype(str)
        q_uniq, q_first, q_local = np.unique(qid, return_index=True, return_inverse=True)
        d_uniq, d_first, d_local = np.unique(did, return_index=True, return_inverse=True)
        q_tok = tokenize_to_arrow(tokenize, [c.query_prefix + t for t in q_text[q_first]], c.max_seq_length,
                                  c.pre_truncate_max_chars_per_token)
        d_tok = tokenize_to_arrow(tokenize, [c.document_prefix + t for t in d_text[d_first]], c.max_seq_length,
                                  c.pre_truncate_max_chars_per_token)
        _write_batch(fs, out_root, first_batch + i, {
            "qid_map.parquet": pa.table({c.pair_query_id_col: q_uniq, c.out_query_id_col: np.arange(len(q_uniq), dtype=np.int32)}),
            "did_map.parquet": pa.table({c.pair_document_id_col: d_uniq, c.out_document_id_col: np.arange(len(d_uniq), dtype=np.int32)}),
            "relations.parquet": pa.table({c.out_query_id_col: q_local.astype(np.int32), c.out_document_id_col: d_local.astype(np.int32),
                                           c.out_relevance_col: np.ones(len(qid), dtype=np.int32)}),
            "queries.parquet": pa.table({c.out_query_id_col: np.arange(len(q_uniq), dtype=np.int32), c.out_query_tokens_col: q_tok}),
            "documents.parquet": pa.table({c.out_document_id_col: np.arange(len(d_uniq), dtype=np.int32), c.out_document_tokens_col: d_tok}),
        })
        written += 1
    logger.info(f"shard {c.shard_info.shard_id}/{c.shard_info.num_shards}: wrote {written} batches to {c.output_dir}")
    return written


def _id_to_text(location: str, id_col: str, text_col: str, max_chars: int) -> dict:
    out = {}
    for t in ParquetCollection.from_location(location).stream_tables([id_col, text_col]):
        for i, s in zip(t[id_col].to_pylist(), t[text_col].to_pylist()):
            out[i] = (s or "")[:max_chars]
    return out


def pretokenize_mined_data(config: MinedDataJob, tokenize: Optional[TokenizeFn] = None) -> int:
    """Pre-tokenise and batch mined (query, positives, hard negatives) data; returns the number of batches written.

    For every use ``u`` of a query its negatives are the ``u``-th of ``num_query_uses`` disjoint random groups drawn
    from its labelled negatives; queries with fewer negatives than ``uses x per-batch`` use what they have."""
    import pyarrow as pa

    c = config
    tokenize = tokenize or load_tokenizer(c.tokenizer_id)
    rng = np.random.default_rng(c.random_seed)
    max_chars = c.max_seq_length * c.pre_truncate_max_chars_per_token
    queries = _id_to_text(c.query_loc, c.in_query_id_col, c.in_query_text_col, max_chars)
    documents = _id_to_text(c.document_loc, c.in_document_id_col, c.in_document_text_col, max_chars)
    labels = ParquetCollection.from_location(c.labels_loc).read_all(
        [c.in_query_id_col, c.in_document_id_col, c.in_label_relation_col])
    l_q = labels[c.in_query_id_col].to_numpy(zero_copy_only=False)
    l_d = labels[c.in_document_id_col].to_numpy(zero_copy_only=False)
    l_r = labels[c.in_label_relation_col].to_numpy(zero_copy_only=False)
    order = np.argsort(l_q, kind="stable")
    uniq_q, starts = np.unique(l_q[order], return_index=True)
    ends = np.append(starts[1:], len(order))
    rows_of = {q: order[a:b] for q, a, b in zip(uniq_q.tolist(), starts, ends)}
    per_repeat = len(uniq_q) // c.queries_per_batch
    if per_repeat == 0:
        raise ValueError(f"{len(uniq_q)} labelled queries cannot fill one batch of {c.queries_per_batch}")
    fs, out_root = filesystem_for(c.output_loc)
    _write_metadata(fs, out_root, {"tokenizer_huggingface_id": c.tokenizer_id, "queries_per_batch": c.queries_per_batch,
                                   "num_query_uses": c.num_query_uses,
                                   "max_negatives_per_query_per_batch": c.num_negatives_per_query_per_batch,
                                   "max_seq_length": c.max_seq_length, "query_prefix": c.query_prefix,
                                   "document_prefix": c.document_prefix})
    data_root = posixpath.join(out_root, "data")
    # one fixed shuffle of every query's negatives, cut into ``num_query_uses`` groups
    neg_groups = {}
    for q, rows in rows_of.items():
        neg = rows[l_r[rows] <= 0]
        pos = rows[l_r[rows] > 0]
        if len(pos) == 0 or len(neg) == 0:
            raise ValueError(f"query {q!r} needs at least one positive and one negative label")
        # most relevant negatives first, so a short budget keeps the hardest ones
        neg = neg[np.argsort(-l_r[neg].astype(np.float64), kind="stable")][: c.num_negatives_per_query_per_batch * c.num_query_uses]
        neg = rng.permutation(neg)
        neg_groups[q] = (pos, [g for g in np.array_split(neg, c.num_query_uses)])
    written = 0
    qid_all = np.array(list(rows_of.keys()), dtype=object)
    for use in range(c.num_query_uses):
        perm = rng.permutation(len(qid_all))[: per_repeat * c.queries_per_batch]
        for b, members in enumerate(np.split(perm, per_repeat)):
            rel_q, rel_d, rel_v = [], [], []
            batch_q = [qid_all[m] for m in members]
            for q in batch_q:
                pos, groups = neg_groups[q]
                chosen_pos = rng.choice(pos, size=min(len(pos), c.max_pos_per_query), replace=False)
                rows = np.concatenate([chosen_pos, groups[use][: c.num_negatives_per_query_per_batch]])
                rel_q.extend([q] * len(rows))
                rel_d.extend(l_d[rows].tolist())
                rel_v.extend(l_r[rows].tolist())
            q_index = {q: i for i, q in enumerate(batch_q)}
            uniq_d = sorted(set(rel_d), key=str)
            d_index = {d: i for i, d in enumerate(uniq_d)}
            q_tok = tokenize_to_arrow(tokenize, [c.query_prefix + queries[q] for q in batch_q], c.max_seq_length,
                                      c.pre_truncate_max_chars_per_token)
            d_tok = tokenize_to_arrow(tokenize, [c.document_prefix + documents[d] for d in uniq_d], c.max_seq_length,
                                      c.pre_truncate_max_chars_per_token)
            _write_batch(fs, data_root, use * per_repeat + b, {
                "relations.parquet": pa.table({c.out_query_id_col: np.array([q_index[q] for q in rel_q], dtype=np.int64),
                                               c.out_document_id_col: np.array([d_index[d] for d in rel_d], dtype=np.int64),
                                               c.out_relevance_col: np.array([1 if v > 0 else -1 for v in rel_v], dtype=np.int64)}),
                "queries.parquet": pa.table({c.out_query_id_col: np.arange(len(batch_q), dtype=np.int64), c.out_query_tokens_col: q_tok}),
                "documents.parquet": pa.table({c.out_document_id_col: np.arange(len(uniq_d), dtype=np.int64), c.out_document_tokens_col: d_tok}),
            })
            written += 1
    logger.info(f"wrote {written} batches to {data_root}")
    return written
