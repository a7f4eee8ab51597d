# SPDX-License-Identifier: Apache-2.0
"""Database description for the prompt: one ``CREATE TABLE`` block per table with column types, comments, example
values, primary and foreign keys — built from the Spider/BIRD ``tables.json`` entry of the database and from values
found in the SQLite file.

Parity: projects/arctic_text2sql_r1/data_preprocessing/process_dataset.py:294-346 (identifier quoting, value sampling),
:443-627 (schema text; in ``train`` mode only key columns, columns the gold answer uses and a random share of the rest
are kept, and the tables are shuffled, so that the model sees varied and incomplete schemas).
"""

from __future__ import annotations

import random
import re
import sqlite3
from typing import Dict
from typing import List
from typing import Optional
from typing import Sequence
from typing import Set

# words that cannot stand unquoted as an identifier in SQLite / common SQL dialects
_RESERVED = set("""
abort action add after all alter analyze and as asc attach autoincrement before begin between by cascade case cast check
collate column commit conflict constraint create cross current_date current_time current_timestamp database default
deferrable deferred delete desc detach distinct drop each else end escape except exclusive exists explain fail for foreign
from full glob group having if ignore immediate in index indexed initially inner insert instead intersect into is isnull
join key left like limit match natural no not notnull null of offset on or order outer plan pragma primary query raise
recursive references regexp reindex release rename replace restrict right rollback row rows savepoint select set table temp
temporary then to transaction trigger union unique update using vacuum values view virtual when where with without
date time year month user role schema position value range rank percent language function top int float double real
char varchar boolean binary blob decimal smallint
""".split())
_PLAIN = re.compile(r"^[A-Za-z_][A-Za-z0-9_]*$")
MAX_VALUE_CHARS = 40
MAX_VALUES_PER_COLUMN = 6
MAX_TRAIN_COLUMNS = 225


def quote_identifier(name: str) -> str:
    """Back-quoted when the name is a reserved word or holds anything but letters, digits and underscores."""
    if name.lower() in _RESERVED or not _PLAIN.match(name):
        return f"`{name}`"
    return name


def sample_column_values(db_file: str, tables: Sequence[str], per_column: int) -> Dict[str, List]:
    """``{"table.column" (lower case): first distinct non-empty values}``; strings are cut to 40 characters."""
    out: Dict[str, List] = {}
    con = sqlite3.connect(f"file:{db_file}?mode=ro", uri=True)
    con.text_factory = lambda b: b.decode(errors="ignore")
    try:
        for table in tables:
            cols = [r[1] for r in con.execute(f"PRAGMA table_info(`{table}`)")]
            for col in cols:
                rows = con.execute(
                    f"SELECT DISTINCT `{col}` FROM `{table}` WHERE `{col}` IS NOT NULL AND `{col}` != '' LIMIT {int(per_column)}"
                ).fetchall()
                vals = [v[0][:MAX_VALUE_CHARS] if isinstance(v[0], str) else v[0] for v in rows]
                if vals:
                    out[f"{table}.{col}".lower()] = vals
    finally:
        con.close()
    return out


def key_columns(db_info: dict) -> Set[int]:
    keys: Set[int] = set()
    for pk in db_info.get("primary_keys", []):
        keys.update(pk if isinstance(pk, list) else [pk])
    for src, dst in db_info.get("foreign_keys", []):
        keys.update((src, dst))
    return keys


def _columns_to_show(db_info: dict, mode: str, answer: str, rng: random.Random) -> Set[int]:
    n = len(db_info["column_names_original"])
    if mode != "train":
        return set(range(n))
    used = set(key_columns(db_info))
    low = (answer or "").lower()
    used.update(i for i, (_, name) in enumerate(db_info["column_names_original"]) if name.lower() in low)
    rest = [i for i in range(n) if i not in used]
    if rest and len(used) < MAX_TRAIN_COLUMNS:
        share = rng.choice([0.1 * k for k in range(1, 11)])
        take = min(int(share * len(rest)), MAX_TRAIN_COLUMNS - len(used))
        used.update(rng.sample(rest, take))
    return used


def describe_database(db_info: dict, sampled_values: Optional[Dict[str, List]] = None,
                      matched_values: Optional[Dict[str, List]] = None, mode: str = "dev", answer: str = "",
                      synthetic_comments: bool = False, rng: Optional[random.Random] = None) -> str:
    """The schema text of one database.  ``matched_values`` (values that occur in the question) are listed before
    ``sampled_values``; at most six examples per column.  ``synthetic_comments``: comments were generated, so a random
    share of them is left out (as real databases lack many)."""
    rng = rng or random.Random(0)
    sampled_values, matched_values = sampled_values or {}, matched_values or {}
    names, comments, types = db_info["column_names_original"], db_info["column_names"], db_info["column_types"]
    if not (len(names) == len(comments) == len(types)):
        raise ValueError("tables.json entry: column name, comment and type lists differ in length")
    show = _columns_to_show(db_info, mode, answer, rng)
    pk_cols = key_cols = None
    blocks = []
    for t_idx, table in enumerate(db_info["table_names_original"]):
        comment_share = rng.choice([0.1 * k for k in range(0, 11)]) if synthetic_comments else 1.0
        lines, pks, fks = [], [], []
        for c_idx, ((owner, col), (_, comment), ctype) in enumerate(zip(names, comments, types)):
            if owner != t_idx or c_idx not in show:
                continue
            key = f"{table}.{col}".lower()
            values = list(dict.fromkeys(list(matched_values.get(key, [])) + list(sampled_values.get(key, []))))[:MAX_VALUES_PER_COLUMN]
            plain = col.lower() in (comment.lower(), comment.lower().replace(" ", "_"), comment.lower().replace(" ", "")) or not comment.strip()
            with_comment = (not plain) and (not synthetic_comments or rng.random() < comment_share)
            line = f"    {quote_identifier(col)} {ctype},"
            if with_comment:
                line += f" -- {comment}" + (f", example: {values}" if values else "")
            elif values:
                line += f" -- example: {values}"
            lines.append(line)
            for pk in db_info.get("primary_keys", []):
                if c_idx in (pk if isinstance(pk, list) else [pk]) and col not in pks:
                    pks.append(col)
            for src, dst in db_info.get("foreign_keys", []):
                if src == c_idx:
                    d_table = db_info["table_names_original"][names[dst][0]]
                    fk = (f"    CONSTRAINT fk_{table.lower().replace(' ', '_')}_{col.lower().replace(' ', '_')} FOREIGN KEY "
                          f"({quote_identifier(col)}) REFERENCES {quote_identifier(d_table)} ({quote_identifier(names[dst][1])}),")
                    if fk not in fks:
                        fks.append(fk)
        if not lines:
            continue
        if pks:
            lines.append("    PRIMARY KEY (" + ", ".join(quote_identifier(c) for c in pks) + "),")
        body = "\n".join(lines + fks)
        if body.endswith(","):
            body = body[:-1]
        blocks.append(f"CREATE TABLE {quote_identifier(table)} (\n{body}\n);")
    if mode == "train":
        rng.shuffle(blocks)
    return "\n\n".join(blocks)


def create_statements(db_file: str) -> List[str]:
    """The ``CREATE TABLE`` statements stored in the SQLite file itself (for databases without a ``tables.json``)."""
    con = sqlite3.connect(f"file:{db_file}?mode=ro", uri=True)
    try:
        return [r[1] for r in con.execute("SELECT name, sql FROM sqlite_master WHERE type='table'") if r[1]]
    finally:
        con.close()


def strip_sql_comments(sql: str) -> str:
    sql = re.sub(r"--.*", "", sql)
    return re.sub(r"/\*.*?\*/", "", sql, flags=re.S).strip()
