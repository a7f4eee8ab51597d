# SPDX-License-Identifier: Apache-2.0
"""Search index over the text cells of a database, used to find the stored values a question refers to.

The reference builds one Lucene BM25 index per database with pyserini (Java) and queries it with all n-grams of the
question (projects/arctic_text2sql_r1/data_preprocessing/build_contents_index.py:66-124, process_dataset.py:348-441).
This is a dependency-free BM25 over the same documents — one per distinct ``(table, column, value)`` — stored as one
JSON file per database; the matching rule on top is the same: a value is kept when at least 85 % of it occurs as a
substring of the question, the 20 best (coverage, then length) survive.
"""

from __future__ import annotations

import json
import math
import re
import sqlite3
from collections import Counter
from collections import defaultdict
from pathlib import Path
from typing import Dict
from typing import List
from typing import Tuple

_TOKEN = re.compile(r"[A-Za-z0-9]+|[^\sA-Za-z0-9]")
MAX_CELL_CHARS = 200


def tokenize(text: str) -> List[str]:
    return [t.lower() for t in _TOKEN.findall(text)]


def n_grams(text: str, max_n: int = 8) -> List[str]:
    """All word n-grams up to ``max_n`` words, joined by single spaces, in order of first appearance."""
    words = _TOKEN.findall(text)
    out = []
    for n in range(1, max_n + 1):
        out.extend(" ".join(words[i : i + n]) for i in range(len(words) - n + 1))
    return list(dict.fromkeys(out))


def _is_number(s: str) -> bool:
    try:
        float(s)
        return True
    except ValueError:
        return False


def collect_text_cells(db_file: str) -> List[dict]:
    """One document per distinct non-numeric text value of every column: ``{"id": "table-**-column-**-n", "contents"}``."""
    con = sqlite3.connect(f"file:{db_file}?mode=ro", uri=True)
    con.text_factory = lambda b: b.decode(errors="ignore")
    docs = []
    try:
        tables = [r[0] for r in con.execute("SELECT name FROM sqlite_master WHERE type='table' AND name != 'sqlite_sequence'")]
        for table in tables:
            for col in [r[1] for r in con.execute(f"PRAGMA table_info(`{table}`)")]:
                try:
                    rows = con.execute(f"SELECT DISTINCT `{col}` FROM `{table}` WHERE `{col}` IS NOT NULL").fetchall()
                except sqlite3.Error:
                    continue
                k = 0
                for (v,) in rows:
                    if isinstance(v, str) and v.strip() and len(v) <= MAX_CELL_CHARS and not _is_number(v.strip()):
                        docs.append({"id": f"{table}-**-{col}-**-{k}", "contents": v})
                        k += 1
    finally:
        con.close()
    return docs


class ValueIndex:
    """BM25 (k1 = 0.9, b = 0.4 — the defaults of the Lucene searcher the reference uses) over short documents."""

    K1, B = 0.9, 0.4

    def __init__(self, docs: List[dict]) -> None:
        self.docs = docs
        self.postings: Dict[str, List[Tuple[int, int]]] = defaultdict(list)
        self.lengths: List[int] = []
        for i, d in enumerate(docs):
            tf = Counter(tokenize(d["contents"]))
            self.lengths.append(sum(tf.values()))
            for tok, c in tf.items():
                self.postings[tok].append((i, c))
        self.avg_len = (sum(self.lengths) / len(self.lengths)) if self.lengths else 1.0

    @classmethod
    def build(cls, db_file: str) -> "ValueIndex":
        return cls(collect_text_cells(db_file))

    def save(self, path) -> None:
        Path(path).parent.mkdir(parents=True, exist_ok=True)
        Path(path).write_text(json.dumps(self.docs, ensure_ascii=False))

    @classmethod
    def load(cls, path) -> "ValueIndex":
        return cls(json.loads(Path(path).read_text()))

    def search(self, query: str, k: int = 10) -> List[dict]:
        scores: Dict[int, float] = defaultdict(float)
        n = len(self.docs)
        for tok in set(tokenize(query)):
            plist = self.postings.get(tok)
            if not plist:
                continue
            idf = math.log(1 + (n - len(plist) + 0.5) / (len(plist) + 0.5))
            for doc, tf in plist:
                norm = tf + self.K1 * (1 - self.B + self.B * self.lengths[doc] / self.avg_len)
                scores[doc] += idf * tf * (self.K1 + 1) / norm
        best = sorted(scores.items(), key=lambda kv: (-kv[1], kv[0]))[:k]
        return [self.docs[i] for i, _ in best]


def substring_coverage(value: str, question: str) -> float:
    """Length of the longest substring of ``value`` that occurs in ``question``, over the length of ``value``."""
    v, q = value.lower(), question.lower()
    if not v:
        return 0.0
    best = 0
    for i in range(len(v)):
        lo = best + 1  # only a longer match matters
        if i + lo > len(v):
            break
        if v[i : i + lo] not in q:
            continue
        j = i + lo
        while j < len(v) and v[i : j + 1] in q:
            j += 1
        best = j - i
    return best / len(v)


def question_values(index: ValueIndex, question: str, threshold: float = 0.85, keep: int = 20, hits_per_query: int = 10
                    ) -> Dict[str, List[str]]:
    """``{"table.column": [values]}`` of stored values the question mentions."""
    seen, hits = set(), []
    for q in n_grams(question, 8) + [question]:
        for h in index.search(q, hits_per_query):
            if h["id"] not in seen:
                seen.add(h["id"])
                hits.append(h)
    scored = []
    for order, h in enumerate(hits):
        table, col, _ = h["id"].split("-**-")
        s = substring_coverage(h["contents"], question)
        if s > threshold:
            scored.append((s, len(h["contents"]), order, f"{table}.{col}".lower(), h["contents"]))
    scored.sort(key=lambda x: (x[0], x[1], x[2]), reverse=True)
    out: Dict[str, List[str]] = {}
    for _, _, _, key, value in scored[:keep]:
        out.setdefault(key, []).append(value)
    return out


def build_indexes(db_root: str, index_root: str) -> List[str]:
    """One ``<db_id>.json`` index per ``<db_root>/<db_id>/<db_id>.sqlite``; returns the database ids."""
    done = []
    for d in sorted(Path(db_root).iterdir()):
        f = d / f"{d.name}.sqlite"
        if f.exists():
            ValueIndex.build(str(f)).save(Path(index_root) / f"{d.name}.json")
            done.append(d.name)
    return done
