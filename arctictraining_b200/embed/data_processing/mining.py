# SPDX-License-Identifier: Apache-2.0
"""Hard-negative mining on top of dense retrieval scores, and the merging of several source datasets.

Parity: projects/arctic_embed/examples/finetune_models/data_processing_scripts/stage_3_mine.py:29-172 (negatives are the
highest-scoring retrieved documents that are not labelled positive and score below ``threshold x`` the score of the
weakest positive that is kept — the guard against unlabelled positives) and stage_4_combine.py:30-93 (ids of different
sources are re-hashed with a per-source offset so that they cannot collide).  The mining here is one vectorised pass
over all (query, retrieved document) rows instead of a Python loop over the queries.
"""

from __future__ import annotations

from typing import Dict
from typing import Sequence
from typing import Tuple

import numpy as np


def mine_hard_negatives(score_q: np.ndarray, score_d: np.ndarray, score: np.ndarray, label_q: np.ndarray, label_d: np.ndarray,
                        threshold: float = 0.95, negatives_per_query: int = 10, max_positives_per_query: int = 1
                        ) -> Tuple[np.ndarray, np.ndarray, np.ndarray, Dict[str, int]]:
    """``(query ids, document ids, relevance)`` rows: per query its ``max_positives_per_query`` best-scoring labelled
    positives (+1) and the ``negatives_per_query`` hardest eligible negatives (-1).  Queries whose positives were not
    retrieved, or with too few eligible negatives, are dropped; the counts are returned as statistics."""
    order = np.lexsort((-score, score_q))                 # by query, best score first
    q, d, s = score_q[order], score_d[order], score[order]
    # labelled positive? membership test on (query, document) pairs via a structured view
    pair = np.empty(len(q), dtype=[("q", q.dtype), ("d", d.dtype)])
    pair["q"], pair["d"] = q, d
    lab = np.empty(len(label_q), dtype=pair.dtype)
    lab["q"], lab["d"] = label_q.astype(q.dtype), label_d.astype(d.dtype)
    is_pos = np.isin(pair, lab)
    uniq, start = np.unique(q, return_index=True)
    seg = np.searchsorted(uniq, q)                         # segment (query) of every row
    # rank of every positive among the positives of its query (rows are score-sorted inside a query)
    pos_rank = np.cumsum(is_pos) - np.concatenate([[0], np.cumsum(is_pos)])[start][seg] - 1
    keep_pos = is_pos & (pos_rank < max_positives_per_query)
    n_pos = np.bincount(seg, weights=is_pos, minlength=len(uniq)).astype(np.int64)
    # score of the weakest kept positive per query = cutoff reference
    weakest = np.full(len(uniq), np.inf)
    np.minimum.at(weakest, seg[keep_pos], s[keep_pos])
    cutoff = threshold * weakest
    eligible = (~is_pos) & (s < cutoff[seg])
    neg_rank = np.cumsum(eligible) - np.concatenate([[0], np.cumsum(eligible)])[start][seg] - 1
    keep_neg = eligible & (neg_rank < negatives_per_query)
    n_neg = np.bincount(seg, weights=keep_neg, minlength=len(uniq)).astype(np.int64)
    good_query = (n_pos > 0) & (n_neg >= negatives_per_query)
    keep = (keep_pos | keep_neg) & good_query[seg]
    rel = np.where(keep_pos, 1, -1).astype(np.int8)
    stats = {"queries": int(len(uniq)), "kept_queries": int(good_query.sum()),
             "dropped_no_positive_retrieved": int((n_pos == 0).sum()),
             "dropped_too_few_negatives": int(((n_pos > 0) & (n_neg < negatives_per_query)).sum()),
             "dropped_extra_positives": int((is_pos & ~keep_pos & good_query[seg]).sum())}
    # positives first inside a query, then negatives by falling score
    out_order = np.lexsort((-s[keep], ~keep_pos[keep], q[keep]))
    return q[keep][out_order], d[keep][out_order], rel[keep][out_order], stats


def scramble_ids(ids: np.ndarray, source_index: int) -> np.ndarray:
    """Deterministic 64-bit re-hash of ``ids`` with an offset that depends on the source: the same id in two sources maps
    to two different values, distinct ids of one source stay distinct (a bijective mixing function)."""
    x = ids.astype(np.uint64) + np.uint64(np.random.default_rng(source_index).integers(1, 2**63, dtype=np.uint64))
    with np.errstate(over="ignore"):  # splitmix64 finaliser: invertible on 64-bit integers
        x ^= x >> np.uint64(30)
        x *= np.uint64(0xBF58476D1CE4E5B9)
        x ^= x >> np.uint64(27)
        x *= np.uint64(0x94D049BB133111EB)
        x ^= x >> np.uint64(31)
    return x


def combine_datasets(tables_per_source: Sequence[Dict[str, "object"]]) -> Dict[str, "object"]:
    """Concatenate the ``queries`` / ``documents`` / ``labels`` tables of several sources after scrambling every
    ``*_ID`` column per source; query and document ids of the result must be unique."""
    import pyarrow as pa

    out = {}
    for name in tables_per_source[0]:
        parts = []
        for i, tables in enumerate(tables_per_source):
            t = tables[name]
            for ci, col in enumerate(t.column_names):
                if col.endswith("ID"):
                    t = t.set_column(ci, col, pa.array(scramble_ids(t.column(col).to_numpy(), i)))
            parts.append(t)
        out[name] = pa.concat_tables(parts)
    for name, col in (("queries", "QUERY_ID"), ("documents", "DOCUMENT_ID")):
        if name in out:
            ids = out[name].column(col).to_numpy()
            if len(np.unique(ids)) != len(ids):
                raise ValueError(f"{col} values collide after combining the sources")
    return out
