# SPDX-License-Identifier: Apache-2.0
"""Execution-based checking of generated SQL against SQLite databases (BIRD / Spider layout: one `<db_id>.sqlite` per
database directory).  A query is run in a worker process with a time limit; results are compared as multisets of rows.
Same role as projects/excot_dpo/utils/sql_exec.py in the reference."""

from __future__ import annotations

import multiprocessing as mp
import re
import sqlite3
from collections import Counter
from pathlib import Path
from typing import Any
from typing import List
from typing import Optional
from typing import Tuple

_SQL_BLOCK = re.compile(r"```sql\s*(.*?)```", re.S | re.I)


def extract_sql(text: str) -> Optional[str]:
    """Last ```sql fenced block of a chain-of-thought answer, or the text after a final 'SQL:' marker."""
    blocks = _SQL_BLOCK.findall(text or "")
    if blocks:
        return blocks[-1].strip().rstrip(";") + ";"
    m = re.search(r"(?:final\s+)?sql\s*:\s*(select.*)$", text or "", re.S | re.I)
    return (m.group(1).strip().rstrip(";") + ";") if m else None


def _run(db_path: str, sql: str, out) -> None:
    try:
        con = sqlite3.connect(f"file:{db_path}?mode=ro", uri=True) if db_path != ":memory:" else sqlite3.connect(db_path)
        con.text_factory = lambda b: b.decode(errors="ignore")
        rows = con.execute(sql).fetchall()
        con.close()
        out.put(("ok", rows))
    except Exception as e:  # noqa: BLE001 - the error text is the result
        out.put(("error", str(e)))


def execute(db_path: str, sql: str, timeout_s: float = 30.0) -> Tuple[str, Any]:
    """Returns ("ok", rows) | ("error", message) | ("timeout", None)."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_run, args=(db_path, sql, q))
    p.start()
    p.join(timeout_s)
    if p.is_alive():
        p.terminate()
        p.join()
        return "timeout", None
    return q.get() if not q.empty() else ("error", "no result")


def same_result(a: List[tuple], b: List[tuple]) -> bool:
    return Counter(map(tuple, a)) == Counter(map(tuple, b))


def database_path(db_root: str, db_id: str) -> str:
    return str(Path(db_root) / db_id / f"{db_id}.sqlite")


def is_correct(db_root: str, db_id: str, predicted_sql: Optional[str], gold_sql: str, timeout_s: float = 30.0) -> bool:
    if not predicted_sql:
        return False
    path = database_path(db_root, db_id)
    s1, r1 = execute(path, predicted_sql, timeout_s)
    if s1 != "ok":
        return False
    s2, r2 = execute(path, gold_sql, timeout_s)
    return s2 == "ok" and same_result(r1, r2)
