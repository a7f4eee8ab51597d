# SPDX-License-Identifier: Apache-2.0
"""Hard-negative mining for contrastive training: embed queries and documents with a teacher model, retrieve the
top-k documents per query by dense dot product, drop the positives and anything scoring above
`max_negative_to_positive_ratio` x the positive's score (likely false negatives), keep the next `num_negatives`.

    python projects/arctic_embed/data_processing/mine_hard_negatives.py --input pairs.jsonl --out mined.jsonl \
        --teacher Snowflake/snowflake-arctic-embed-m-v1.5 --num-negatives 10

The reference spreads these steps over data_processing_scripts/stage_{1_embed,2_score_and_retrieve,3_mine}.py and
data_processing/dense_retrieval.py.
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path
from typing import List

import torch


@torch.no_grad()
def embed_texts(model, tok, texts: List[str], batch_size: int, max_len: int, device) -> torch.Tensor:
    out = []
    for i in range(0, len(texts), batch_size):
        enc = tok(texts[i : i + batch_size], padding=True, truncation=True, max_length=max_len, return_tensors="pt").to(device)
        hidden = model(**enc).last_hidden_state[:, 0]  # first-token pooling
        out.append(torch.nn.functional.normalize(hidden.float(), dim=-1).cpu())
    return torch.cat(out)


def dense_retrieve(q: torch.Tensor, d: torch.Tensor, k: int, chunk: int = 1024):
    """Top-k document indices and scores per query, computed in query chunks."""
    scores, idx = [], []
    for i in range(0, q.shape[0], chunk):
        s = q[i : i + chunk] @ d.T
        top = torch.topk(s, min(k, d.shape[0]), dim=-1)
        scores.append(top.values)
        idx.append(top.indices)
    return torch.cat(idx), torch.cat(scores)


def mine(rows: List[dict], q: torch.Tensor, d: torch.Tensor, doc_of_row: List[int], num_negatives: int, k: int,
         max_ratio: float) -> List[dict]:
    idx, scores = dense_retrieve(q, d, k)
    docs = [None] * d.shape[0]
    for r, di in zip(rows, doc_of_row):
        docs[di] = r["document"]
    out = []
    for qi, r in enumerate(rows):
        pos = doc_of_row[qi]
        pos_score = float(q[qi] @ d[pos])
        negs = [docs[int(j)] for j, s in zip(idx[qi], scores[qi]) if int(j) != pos and float(s) <= max_ratio * pos_score]
        out.append({**r, "negatives": negs[:num_negatives]})
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--input", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--teacher", required=True)
    ap.add_argument("--num-negatives", type=int, default=10)
    ap.add_argument("--top-k", type=int, default=100)
    ap.add_argument("--max-negative-to-positive-ratio", type=float, default=0.95)
    ap.add_argument("--batch-size", type=int, default=128)
    args = ap.parse_args()

    from transformers import AutoModel
    from transformers import AutoTokenizer

    rows = [json.loads(line) for line in Path(args.input).read_text().splitlines() if line.strip()]
    device = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    tok = AutoTokenizer.from_pretrained(args.teacher)
    model = AutoModel.from_pretrained(args.teacher).to(device).eval()
    uniq, doc_of_row = {}, []
    for r in rows:
        doc_of_row.append(uniq.setdefault(r["document"], len(uniq)))
    q = embed_texts(model, tok, [r["query"] for r in rows], args.batch_size, 64, device)
    d = embed_texts(model, tok, list(uniq), args.batch_size, 512, device)
    mined = mine(rows, q, d, doc_of_row, args.num_negatives, args.top_k, args.max_negative_to_positive_ratio)
    with open(args.out, "w") as f:
        for r in mined:
            f.write(json.dumps(r) + "\n")
    print(f"{len(mined)} queries with up to {args.num_negatives} mined negatives -> {args.out}")


if __name__ == "__main__":
    main()
