# SPDX-License-Identifier: Apache-2.0
"""BIRD evaluation for text-to-SQL models: sample n answers per question with vLLM, take the final SQL of each, vote by
execution result (self-consistency) and report execution accuracy.  Training code for this project is not part of the
reference either (projects/arctic_text2sql_r1/README.md:14); its bird_eval/ directory has the same three stages.

    python projects/arctic_text2sql_r1/bird_eval.py --model <path> --questions dev.json --schemas schemas.json \
        --db-root dev_databases --n 8 --out preds.jsonl
"""

from __future__ import annotations

import argparse
import json
import sys
from collections import Counter
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent / "excot_dpo"))

from excot.prompts import build_messages  # noqa: E402
from excot.sql_exec import database_path  # noqa: E402
from excot.sql_exec import execute  # noqa: E402
from excot.sql_exec import extract_sql  # noqa: E402
from excot.sql_exec import same_result  # noqa: E402


def vote(db_path: str, sqls: list, timeout_s: float):
    """Self-consistency: the SQL whose execution result is shared by most samples (ties: first seen)."""
    results, keys = [], []
    for s in sqls:
        status, rows = execute(db_path, s, timeout_s) if s else ("error", None)
        results.append(rows if status == "ok" else None)
        keys.append(None if status != "ok" else tuple(sorted(map(repr, rows))))
    counts = Counter(k for k in keys if k is not None)
    if not counts:
        return None, None
    best = counts.most_common(1)[0][0]
    i = keys.index(best)
    return sqls[i], results[i]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--questions", required=True)
    ap.add_argument("--schemas", required=True)
    ap.add_argument("--db-root", required=True)
    ap.add_argument("--n", type=int, default=8)
    ap.add_argument("--temperature", type=float, default=0.8)
    ap.add_argument("--timeout", type=float, default=30.0)
    ap.add_argument("--out", default="preds.jsonl")
    args = ap.parse_args()

    from vllm import SamplingParams

    from arctictraining_b200.synth import VllmSynth

    questions = json.loads(Path(args.questions).read_text())
    schemas = json.loads(Path(args.schemas).read_text())
    client = VllmSynth(model_params={"model": args.model},
                       sampling_params=SamplingParams(temperature=args.temperature, max_tokens=2048, n=args.n))
    ids = {}
    for i, q in enumerate(questions):
        msgs = build_messages(schemas[q["db_id"]], q["question"], q.get("evidence", ""))
        ids[client.add_chat_to_batch_task("bird", messages=msgs)] = i
    answers = {ids[o["custom_id"]]: [c["content"] for c in o["choices"]]
               for o in client.extract_messages_from_responses(client.execute_batch_task("bird"))}
    correct = 0
    with open(args.out, "w") as f:
        for i, q in enumerate(questions):
            path = database_path(args.db_root, q["db_id"])
            sql, rows = vote(path, [extract_sql(a) for a in answers.get(i, [])], args.timeout)
            status, gold = execute(path, q.get("SQL") or q.get("query"), args.timeout)
            ok = bool(sql) and status == "ok" and rows is not None and same_result(rows, gold)
            correct += ok
            f.write(json.dumps({"qid": i, "db_id": q["db_id"], "pred_sql": sql, "correct": ok}) + "\n")
    print(json.dumps({"questions": len(questions), "execution_accuracy": correct / max(1, len(questions))}))


if __name__ == "__main__":
    main()
