# SPDX-License-Identifier: Apache-2.0
"""Turn (query, document, relevance) data into the pre-tokenised, pre-batched parquet layout that the biencoder
trainer streams (`arctictraining_b200/embed/data.py`): one `batch_XXXXXXXX/` directory per global batch with
`queries.parquet`, `documents.parquet` and `relations.parquet`.

Two input kinds, as in the reference's projects/arctic_embed/src/arctic_embed/data_processing/pretokenize.py:
* pairs: a JSONL / parquet file with `query`, `document` columns (in-batch negatives only);
* mined: additionally `negatives` (list of hard-negative documents per query, e.g. from `mine_hard_negatives.py`).

    python projects/arctic_embed/data_processing/pretokenize.py --input pairs.jsonl --out data/train \
        --tokenizer intfloat/e5-base-unsupervised --batch-size 256 --query-prefix "query: " --document-prefix "passage: "
"""

from __future__ import annotations

import argparse
import json
import random
from pathlib import Path
from typing import Dict
from typing import List

import pyarrow as pa
import pyarrow.parquet as pq


def read_rows(path: str) -> List[dict]:
    if path.endswith(".parquet"):
        return pq.read_table(path).to_pylist()
    return [json.loads(line) for line in Path(path).read_text().splitlines() if line.strip()]


def write_batch(out_dir: Path, index: int, queries: List[List[int]], documents: List[List[int]], relations: List[tuple]) -> None:
    d = out_dir / f"batch_{index:08d}"
    d.mkdir(parents=True, exist_ok=True)
    pq.write_table(pa.table({"BATCH_QUERY_ID": list(range(len(queries))), "QUERY_TOKEN_ID_LIST": queries}), d / "queries.parquet")
    pq.write_table(pa.table({"BATCH_DOCUMENT_ID": list(range(len(documents))), "DOCUMENT_TOKEN_ID_LIST": documents}),
                   d / "documents.parquet")
    pq.write_table(pa.table({"BATCH_QUERY_ID": [r[0] for r in relations], "BATCH_DOCUMENT_ID": [r[1] for r in relations],
                             "RELEVANCE": [r[2] for r in relations]}), d / "relations.parquet")


def build_batches(rows: List[dict], tokenize, batch_size: int, negatives_per_query: int, seed: int, out_dir: Path,
                  drop_last: bool = True) -> int:
    """Shuffle, cut into global batches of `batch_size` queries, de-duplicate documents inside a batch (a document
    shared by two queries is stored once and is relevant to both) and write one directory per batch."""
    rng = random.Random(seed)
    rows = list(rows)
    rng.shuffle(rows)
    n_written = 0
    for start in range(0, len(rows), batch_size):
        chunk = rows[start : start + batch_size]
        if len(chunk) < batch_size and drop_last:
            break
        doc_index: Dict[str, int] = {}
        docs: List[str] = []
        relations = []
        for qi, r in enumerate(chunk):
            texts = [(r["document"], 1)] + [(n, -1) for n in (r.get("negatives") or [])[:negatives_per_query]]
            for text, rel in texts:
                di = doc_index.setdefault(text, len(docs))
                if di == len(docs):
                    docs.append(text)
                relations.append((qi, di, rel))
        write_batch(out_dir, n_written, tokenize([r["query"] for r in chunk], True), tokenize(docs, False), relations)
        n_written += 1
    return n_written


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--input", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--tokenizer", required=True)
    ap.add_argument("--batch-size", type=int, default=256)
    ap.add_argument("--negatives-per-query", type=int, default=0)
    ap.add_argument("--max-query-len", type=int, default=32)
    ap.add_argument("--max-document-len", type=int, default=256)
    ap.add_argument("--query-prefix", default="")
    ap.add_argument("--document-prefix", default="")
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args()

    from transformers import AutoTokenizer

    tok = AutoTokenizer.from_pretrained(args.tokenizer)

    def tokenize(texts: List[str], is_query: bool) -> List[List[int]]:
        prefix = args.query_prefix if is_query else args.document_prefix
        limit = args.max_query_len if is_query else args.max_document_len
        return tok([prefix + t for t in texts], truncation=True, max_length=limit, add_special_tokens=True)["input_ids"]

    n = build_batches(read_rows(args.input), tokenize, args.batch_size, args.negatives_per_query, args.seed, Path(args.out))
    print(f"wrote {n} batches of {args.batch_size} queries to {args.out}")


if __name__ == "__main__":
    main()
