# SPDX-License-Identifier: Apache-2.0
"""Fetch a public retrieval dataset and write it in the layout `prepare_data.py` starts from:

    <out>/<name>/queries.parquet    QUERY_ID, QUERY_TEXT
    <out>/<name>/documents.parquet  DOCUMENT_ID, DOCUMENT_TEXT
    <out>/<name>/labels.parquet     QUERY_ID, DOCUMENT_ID       (the annotated positives)

    python download_data.py nq msmarco hotpotqa stackexchange fever --out data

Ids are 64-bit hashes of the text, so equal texts collapse to one row and the same text gets the same id in every
run.  Needs network access to the Hugging Face hub (and to fever.ai for `fever`).

Sources of the reference: projects/arctic_embed/examples/finetune_models/data_download_scripts/download_*.py.
"""

from __future__ import annotations

import argparse
import hashlib
from pathlib import Path
from typing import Callable
from typing import Dict
from typing import Iterable
from typing import Optional
from typing import Sequence
from typing import Tuple

import numpy as np
import pyarrow as pa
import pyarrow.parquet as pq


def text_ids(texts: Sequence[str]) -> np.ndarray:
    """Stable unsigned 64-bit id of every text (first 8 bytes of its BLAKE2b digest)."""
    out = np.empty(len(texts), dtype=np.uint64)
    for i, t in enumerate(texts):
        out[i] = int.from_bytes(hashlib.blake2b(t.encode("utf-8"), digest_size=8).digest(), "little")
    return out


def pairs_to_tables(queries: Sequence[str], documents: Sequence[str],
                    extra_documents: Optional[Sequence[str]] = None) -> Dict[str, pa.Table]:
    """Tables of a list of (query, positive document) pairs.  Queries and documents are de-duplicated by text, the
    labels by pair; `extra_documents` (a corpus without labels, e.g. all passages of a collection) join the documents."""
    if len(queries) != len(documents):
        raise ValueError("one positive document per query text is expected")
    q_text = np.asarray(queries, dtype=object)
    d_text = np.asarray(documents, dtype=object)
    qid, did = text_ids(q_text), text_ids(d_text)
    uq, qi = np.unique(qid, return_index=True)
    all_d_text, all_did = d_text, did
    if extra_documents is not None and len(extra_documents):
        extra = np.asarray(extra_documents, dtype=object)
        all_d_text = np.concatenate([d_text, extra])
        all_did = np.concatenate([did, text_ids(extra)])
    ud, di = np.unique(all_did, return_index=True)
    pairs = np.unique(np.stack([qid, did], axis=1), axis=0)
    return {
        "queries": pa.table({"QUERY_ID": uq, "QUERY_TEXT": pa.array(q_text[qi].tolist(), pa.string())}),
        "documents": pa.table({"DOCUMENT_ID": ud, "DOCUMENT_TEXT": pa.array(all_d_text[di].tolist(), pa.string())}),
        "labels": pa.table({"QUERY_ID": pairs[:, 0], "DOCUMENT_ID": pairs[:, 1]}),
    }


def write_tables(tables: Dict[str, pa.Table], out_dir: Path) -> None:
    out_dir.mkdir(parents=True, exist_ok=True)
    for name, table in tables.items():
        pq.write_table(table, out_dir / f"{name}.parquet")
    print(f"{out_dir}: {len(tables['queries']):,} queries, {len(tables['documents']):,} documents, "
          f"{len(tables['labels']):,} labels")


def title_and_text(title: str, text: str) -> str:
    """Document text of a titled passage: the title on its own line when there is one."""
    title, text = (title or "").strip(), (text or "").strip()
    return f"{title}\n{text}" if title else text


class BodyIndex:
    """Find which known body text a 'title body' string ends with.  Bodies are bucketed by their last `key` characters,
    so a look-up compares against the few bodies that share the tail instead of all of them."""

    def __init__(self, bodies: Iterable[str], key: int = 32):
        self.key = key
        self.buckets: Dict[str, list] = {}
        for body in bodies:
            if body:
                self.buckets.setdefault(body[-key:], []).append(body)
        self.short_lengths = sorted({len(k) for k in self.buckets if len(k) < key})  # bodies shorter than the key

    def split(self, combo: str) -> Optional[Tuple[str, str]]:
        """(title, body) with `body` the longest known body that `combo` ends with; None when there is none."""
        best = None
        for n in {min(self.key, len(combo)), *(m for m in self.short_lengths if m <= len(combo))}:
            for body in self.buckets.get(combo[-n:], ()):
                if combo.endswith(body) and (best is None or len(body) > len(best)):
                    best = body
        if best is None:
            return None
        return combo[:len(combo) - len(best)].rstrip(), best


# ---------------------------------------------------------------------------------------------------------------------
# one loader per dataset: returns (query texts, positive document texts, extra corpus documents or None)

def _load_nq():
    from datasets import load_dataset

    d = load_dataset("sentence-transformers/natural-questions", split="train")
    return d["query"], d["answer"], None


def _load_hotpotqa():
    from datasets import load_dataset

    d = load_dataset("sentence-transformers/hotpotqa", "triplet-all", split="train").to_pandas()
    d = d.drop_duplicates(subset=["anchor", "positive"])
    extra = d["negative"].drop_duplicates().tolist()  # the annotated negatives stay in the corpus as distractors
    return d["anchor"].tolist(), d["positive"].tolist(), extra


def _load_msmarco():
    from datasets import load_dataset

    corpus = load_dataset("Tevatron/msmarco-passage-corpus", split="train")
    extra = [title_and_text(t, x) for t, x in zip(corpus["title"], corpus["text"])]
    train = load_dataset("Tevatron/msmarco-passage", split="train")
    queries, docs = [], []
    for row in train:
        for p in row["positive_passages"]:
            queries.append(row["query"])
            docs.append(title_and_text(p.get("title", ""), p["text"]))
    return queries, docs, extra


def _load_stackexchange():
    """Duplicate-question pairs: the title of one question retrieves the body of its duplicate and the other way
    round.  The pair file glues title and body together; the bodies alone come from the body-body variant of the
    dataset, and the title is what stands in front of the body."""
    import pandas as pd
    from datasets import load_dataset

    url = ("https://huggingface.co/datasets/sentence-transformers/embedding-training-data/resolve/main/"
           "stackexchange_duplicate_questions_title-body_title-body.jsonl.gz")
    pairs = pd.read_json(url, lines=True)
    bodies = load_dataset("sentence-transformers/stackexchange-duplicates", name="body-body-pair", split="train")
    index = BodyIndex(list(bodies["body1"]) + list(bodies["body2"]))
    queries, docs, lost = [], [], 0
    for a, b in zip(pairs.iloc[:, 0], pairs.iloc[:, 1]):
        ra, rb = index.split(a), index.split(b)
        if ra is None or rb is None:
            lost += 1
            continue
        queries += [ra[0], rb[0]]
        docs += [rb[1], ra[1]]
    print(f"stackexchange: {lost:,} pairs dropped (body not found)")
    return queries, docs, None


def _load_fever():
    """Claims that are supported or refuted, each paired with the Wikipedia pages of its evidence."""
    import io
    import json
    import urllib.request
    import zipfile

    import pandas as pd

    with urllib.request.urlopen("https://fever.ai/download/fever/wiki-pages.zip") as r:
        archive = zipfile.ZipFile(io.BytesIO(r.read()))
    pages: Dict[str, str] = {}
    for member in archive.namelist():
        if not member.endswith(".jsonl"):
            continue
        for line in archive.read(member).decode("utf-8").splitlines():
            row = json.loads(line)
            if row.get("id") and row.get("text"):
                pages[row["id"]] = title_and_text(row["id"].replace("_", " "), row["text"])
    facts = pd.read_json("https://fever.ai/download/fever/train.jsonl", lines=True)
    queries, docs = [], []
    for claim, label, evidence in zip(facts["claim"], facts["label"], facts["evidence"]):
        if label == "NOT ENOUGH INFO":
            continue
        for page in {e[2] for group in evidence for e in group if e[2] is not None}:
            if page in pages:
                queries.append(claim)
                docs.append(pages[page])
    return queries, docs, list(pages.values())


LOADERS: Dict[str, Callable[[], Tuple[Sequence[str], Sequence[str], Optional[Sequence[str]]]]] = {
    "nq": _load_nq, "hotpotqa": _load_hotpotqa, "msmarco": _load_msmarco, "stackexchange": _load_stackexchange,
    "fever": _load_fever,
}


def main(argv: Optional[Sequence[str]] = None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("datasets", nargs="+", choices=sorted(LOADERS))
    ap.add_argument("--out", default=str(Path(__file__).resolve().parent / "data"))
    args = ap.parse_args(argv)
    for name in args.datasets:
        queries, docs, extra = LOADERS[name]()
        write_tables(pairs_to_tables(queries, docs, extra), Path(args.out) / name)


if __name__ == "__main__":
    main()
