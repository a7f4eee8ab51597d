# SPDX-License-Identifier: Apache-2.0
"""Model input / target pairs for text-to-SQL training and evaluation.

Parity: projects/arctic_text2sql_r1/data_preprocessing/process_dataset.py:414-441 (prompt), :642-802 (which field holds
the answer and the external knowledge for every benchmark).
"""

from __future__ import annotations

import json
import os
import random
from typing import Dict
from typing import List
from typing import Optional

from .schema import describe_database
from .schema import sample_column_values
from .value_index import ValueIndex
from .value_index import question_values

PROMPT = """Task Overview:
You are a data science expert. Below, you are provided with a database schema and a natural language question. Your task is to understand the schema and generate a valid SQL query to answer the question.

Database Engine:
{engine}

Database Schema:
{schema}
This schema describes the database's structure, including tables, columns, primary keys, foreign keys, and any relevant relationships or constraints.

Question:
{question}

Instructions:
- Make sure you only output the information that is asked in the question. If the question asks for a specific column, make sure to only include that column in the SELECT clause, nothing more.
- The generated query should return all of the information asked in the question without any missing or extra information.
- Before generating the final SQL query, please think through the steps of how to write the query.

Output Format:
In your answer, please enclose the generated SQL query in a code block:
```sql
-- Your SQL query
```

Take a deep breath and think step by step to find the correct SQL query.
"""

# benchmark -> (field with the answer in train mode, in dev/test mode, field with external knowledge or None)
SOURCES = {
    "synthetic": ("cot", "cot", "external_knowledge"),
    "bird": ("cot", "SQL", "evidence"),
    "spider": ("cot", "query", None),
    "spider2.0": (None, None, "external_knowledge"),
    "spider_dk": ("query", "query", None),
    "spider_realistic": ("query", "query", None),
    "spider_syn": ("query", "query", None),
    "ehrsql": ("query", "query", None),
    "sciencebenchmark": ("query", "query", None),
}


def full_question(row: dict, source: str) -> str:
    ek_field = SOURCES[source][2]
    ek = (row.get(ek_field) or "").strip() if ek_field else ""
    q = row["SpiderSynQuestion"] if source == "spider_syn" else row["question"]
    return f"{ek}\n{q}" if ek else q


def build_examples(rows: List[dict], tables: List[dict], db_root: str, source: str, mode: str = "dev", values_per_column: int = 2,
                   index_root: Optional[str] = None, seed: int = 42) -> List[dict]:
    """``[{"input_seq", "output_seq", "db_desc", "question", "db_id"}]`` for every row of a benchmark file."""
    if source not in SOURCES:
        raise ValueError(f"unknown source {source!r}; known: {sorted(SOURCES)}")
    if mode not in ("train", "dev", "test"):
        raise ValueError("mode must be train, dev or test")
    rng = random.Random(seed)
    answer_field = SOURCES[source][0 if mode == "train" else 1]
    info = {t["db_id"]: t for t in tables}
    sampled: Dict[str, dict] = {}
    indexes: Dict[str, ValueIndex] = {}
    out = []
    for row in rows:
        db_id = row["db_id"]
        db_file = os.path.join(db_root, db_id, f"{db_id}.sqlite")
        if db_id not in sampled:
            sampled[db_id] = sample_column_values(db_file, info[db_id]["table_names_original"], values_per_column)
            if index_root:
                path = os.path.join(index_root, f"{db_id}.json")
                indexes[db_id] = ValueIndex.load(path) if os.path.exists(path) else ValueIndex.build(db_file)
        question = full_question(row, source)
        matched = question_values(indexes[db_id], question) if db_id in indexes else {}
        answer = row.get(answer_field, "") if answer_field else ""
        desc = describe_database(info[db_id], sampled[db_id], matched, mode=mode, answer=answer,
                                 synthetic_comments=(source == "synthetic"), rng=rng)
        out.append({"input_seq": PROMPT.format(engine="SQLite", schema=desc, question=question), "output_seq": answer,
                    "db_desc": desc, "question": question, "db_id": db_id})
    return out


def write_examples(examples: List[dict], path: str) -> None:
    with open(path, "w", encoding="utf-8") as f:
        f.write(json.dumps(examples, indent=2, ensure_ascii=False))
