# SPDX-License-Identifier: Apache-2.0
"""Execution accuracy of a prediction file against a gold benchmark file.

    python projects/arctic_text2sql_r1/evaluate_bird.py --pred preds.json --gold dev.json --db_path dev_databases \\
        --mode major_voting [--voting soft]

Modes: ``greedy_search`` (first sample), ``major_voting`` (self-consistency over all samples), ``pass@k``.
"""

import argparse
import json
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))

from text2sql.evaluate import load_json  # noqa: E402
from text2sql.evaluate import run_eval  # noqa: E402

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--pred", required=True)
    ap.add_argument("--gold", required=True)
    ap.add_argument("--db_path", required=True)
    ap.add_argument("--mode", default="greedy_search", choices=["greedy_search", "major_voting", "pass@k"])
    ap.add_argument("--voting", default="exact", choices=["exact", "soft"])
    ap.add_argument("--num_cpus", type=int, default=8)
    ap.add_argument("--timeout", type=float, default=10.0)
    ap.add_argument("--save_pred_sqls", action="store_true")
    args = ap.parse_args()
    acc, chosen = run_eval(load_json(args.gold), load_json(args.pred), args.db_path, args.mode, args.num_cpus, args.timeout,
                           args.voting)
    print(json.dumps({"mode": args.mode, "execution_accuracy": acc}))
    if args.save_pred_sqls and chosen is not None:
        Path(args.pred[:-5] + f"_pred_{args.mode}_sqls.json").write_text(json.dumps(chosen, indent=2, ensure_ascii=False))
