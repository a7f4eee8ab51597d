# SPDX-License-Identifier: Apache-2.0
"""Execution accuracy of predicted SQL: greedy, self-consistency voting over samples, pass@k.

Parity: projects/arctic_text2sql_r1/bird_eval/evaluate_bird.py:55-376 and self_consistency.py:23-125.  Queries run in
a pool of worker processes, each under a time limit; a prediction is correct when its set of rows equals that of the
gold query.  Voting: ``exact`` — most frequent result set among the valid samples; ``soft`` — the sample whose result
is most similar to all others, where similarity of two results is the column-wise overlap of their value counts.
"""

from __future__ import annotations

import json
import multiprocessing as mp
import os
import random
import re
import sqlite3
from collections import Counter
from typing import Any
from typing import Dict
from typing import List
from typing import Optional
from typing import Sequence
from typing import Tuple

_BLOCK = re.compile(r"```sql\s*(.*?)```", re.S | re.I)
ERROR_SQL = "Error SQL"


def parse_response(text: str) -> str:
    """The last ```sql block of an answer (comments kept out), or ``""``."""
    blocks = _BLOCK.findall(text or "")
    return blocks[-1].strip() if blocks else ""


def _worker(job: Tuple[int, str, str, float]):
    idx, db_file, sql, timeout = job
    import threading

    result: Dict[str, Any] = {"data_idx": idx, "sql": sql, "valid": 0, "rows": None, "columns": None}
    if not sql or sql == ERROR_SQL:
        return result
    try:
        con = sqlite3.connect(f"file:{db_file}?mode=ro", uri=True)
        con.text_factory = lambda b: b.decode(errors="ignore")
        timer = threading.Timer(timeout, con.interrupt)  # SQLite aborts the running statement
        timer.start()
        try:
            cur = con.execute(sql)
            rows = cur.fetchall()
            result.update(valid=1, rows=rows, columns=[d[0] for d in (cur.description or [])])
        finally:
            timer.cancel()
            con.close()
    except Exception:  # noqa: BLE001 - any failure marks the query invalid
        pass
    return result


def execute_many(db_files: Sequence[str], sqls: Sequence[str], num_cpus: int = 8, timeout: float = 10.0) -> List[dict]:
    jobs = [(i, db, sql, timeout) for i, (db, sql) in enumerate(zip(db_files, sqls))]
    if num_cpus <= 1 or len(jobs) < 4:
        return [_worker(j) for j in jobs]
    with mp.get_context("spawn").Pool(num_cpus) as pool:
        return sorted(pool.map(_worker, jobs, chunksize=8), key=lambda r: r["data_idx"])


def same_rows(a: Optional[List[tuple]], b: Optional[List[tuple]]) -> bool:
    return a is not None and b is not None and set(map(tuple, a)) == set(map(tuple, b))


def soft_similarity(a: Optional[dict], b: Optional[dict]) -> float:
    """Column-wise overlap of value counts of two results (``{"columns", "rows"}``), in [0, 1]."""
    if not a or not b or not a["rows"] or not b["rows"]:
        return 0.0

    def counts(res):
        out: Dict[str, Counter] = {}
        for c, name in enumerate(res["columns"]):
            col = Counter(repr(r[c]) if not isinstance(r[c], (int, float, str, type(None))) else r[c] for r in res["rows"])
            out[name] = out.get(name, Counter()) + col
        return out

    ca, cb = counts(a), counts(b)
    real = possible = 0.0
    for name in set(ca) | set(cb):
        x, y = ca.get(name), cb.get(name)
        if not x or not y:
            possible += sum((x or y).values())
            continue
        for v in set(x) | set(y):
            possible += max(x[v], y[v])
            real += min(x[v], y[v])  # = max - |difference|
    return real / possible if possible else 0.0


def vote(samples: List[dict], method: str = "exact", rng: Optional[random.Random] = None, random_when_all_fail: bool = True) -> str:
    """The SQL chosen among the executed samples of one question."""
    valid = [s for s in samples if s["valid"]]
    if not valid:
        return (rng or random).choice(samples)["sql"] if (random_when_all_fail and samples) else ERROR_SQL
    if method == "exact":
        tally: Dict[Any, List] = {}
        for s in valid:
            key = frozenset(map(tuple, s["rows"]))
            tally.setdefault(key, [0, s["sql"]])[0] += 1
        return max(tally.values(), key=lambda t: t[0])[1]
    if method == "soft":
        best, best_score = valid[0]["sql"], -1.0
        for i, s in enumerate(samples):
            if not s["valid"]:
                continue
            score = 1.0 + sum(soft_similarity(s, o) for j, o in enumerate(samples) if j != i)
            if score > best_score:
                best, best_score = s["sql"], score
        return best
    raise ValueError("voting method must be 'exact' or 'soft'")


def db_file_of(db_root: str, db_id: str) -> str:
    return os.path.join(db_root, db_id, f"{db_id}.sqlite")


def run_eval(gold: List[dict], predictions: List[dict], db_root: str, mode: str = "greedy_search", num_cpus: int = 8,
             timeout: float = 10.0, voting: str = "exact", seed: int = 0) -> Tuple[float, Optional[List[str]]]:
    """``predictions[i]["pred_sqls"]`` holds the sampled SQL of question ``i``.  Returns (accuracy, chosen SQL)."""
    if len(gold) != len(predictions):
        raise ValueError("gold and prediction files differ in length")
    gold_sql = [g.get("SQL") or g.get("query") for g in gold]
    dbs = [db_file_of(db_root, g["db_id"]) for g in gold]
    gold_res = execute_many(dbs, gold_sql, num_cpus, timeout)

    def accuracy(chosen: List[str]) -> List[int]:
        res = execute_many(dbs, chosen, num_cpus, timeout)
        return [int(r["valid"] and g["valid"] and same_rows(r["rows"], g["rows"])) for r, g in zip(res, gold_res)]

    if mode == "greedy_search":
        chosen = [p["pred_sqls"][0] for p in predictions]
        ok = accuracy(chosen)
        return sum(ok) / max(1, len(ok)), chosen
    k = len(predictions[0]["pred_sqls"])
    if mode == "major_voting":
        flat_db = [d for d in dbs for _ in range(k)]
        flat_sql = [s for p in predictions for s in p["pred_sqls"]]
        res = execute_many(flat_db, flat_sql, num_cpus, timeout)
        rng = random.Random(seed)
        chosen = [vote(res[i : i + k], voting, rng) for i in range(0, len(res), k)]
        ok = accuracy(chosen)
        return sum(ok) / max(1, len(ok)), chosen
    if mode == "pass@k":
        per_sample = [accuracy([p["pred_sqls"][j] for p in predictions]) for j in range(k)]
        hit = [int(any(col)) for col in zip(*per_sample)]
        return sum(hit) / max(1, len(hit)), None
    raise ValueError("mode must be greedy_search, major_voting or pass@k")


def load_json(path: str):
    with open(path, encoding="utf-8") as f:
        return json.load(f)
