# SPDX-License-Identifier: Apache-2.0
"""ExCoT data pipeline: generate chain-of-thought answers, verify them by execution, sample SFT and DPO sets, evaluate.

    python -m excot.pipeline generate --questions dev.json --schemas schemas.json --out cand.jsonl --model <name> --n 8
    python -m excot.pipeline verify   --candidates cand.jsonl --db-root databases --out verified.jsonl
    python -m excot.pipeline sft      --verified verified.jsonl --out /data/excot_sft
    python -m excot.pipeline dpo      --verified verified.jsonl --out /data/excot_dpo
    python -m excot.pipeline evaluate --verified verified.jsonl

(run from projects/excot_dpo).  `generate` goes through the batch clients of `arctictraining_b200.synth` (vLLM in
process by default, `--client azure` for the Azure OpenAI batch API).  The reference splits these stages over
projects/excot_dpo/data_generation/*.py and evalution/*.py.
"""

from __future__ import annotations

import argparse
import json
import random
from collections import defaultdict
from pathlib import Path
from typing import Dict
from typing import Iterable
from typing import List

from .prompts import build_messages
from .sql_exec import extract_sql
from .sql_exec import is_correct


def _read_jsonl(path: str) -> List[dict]:
    return [json.loads(line) for line in Path(path).read_text().splitlines() if line.strip()]


def _write_jsonl(path: str, rows: Iterable[dict]) -> None:
    with open(path, "w") as f:
        for r in rows:
            f.write(json.dumps(r) + "\n")


def generate(args) -> None:
    questions = json.loads(Path(args.questions).read_text())
    schemas: Dict[str, str] = json.loads(Path(args.schemas).read_text())
    if args.client == "azure":
        from arctictraining_b200.synth import AzureOpenAISynth

        client = AzureOpenAISynth(work_dir=args.work_dir, credential_path=args.credentials)
        extra = {"model": args.model, "n": args.n, "temperature": args.temperature}
    else:
        from vllm import SamplingParams

        from arctictraining_b200.synth import VllmSynth

        client = VllmSynth(model_params={"model": args.model}, work_dir=args.work_dir,
                           sampling_params=SamplingParams(temperature=args.temperature, max_tokens=2048, n=args.n))
        extra = {}
    ids = {}
    for i, q in enumerate(questions):
        msgs = build_messages(schemas[q["db_id"]], q["question"], q.get("evidence", ""))
        ids[client.add_chat_to_batch_task("excot", messages=msgs, **extra)] = i
    outputs = client.extract_messages_from_responses(client.execute_batch_task("excot"))
    by_id = defaultdict(list)
    for o in outputs:
        by_id[ids[o["custom_id"]]].extend(c["content"] for c in o["choices"])
    rows = []
    for i, q in enumerate(questions):
        for text in by_id.get(i, []):
            rows.append({"qid": i, "db_id": q["db_id"], "question": q["question"], "evidence": q.get("evidence", ""),
                         "gold_sql": q.get("SQL") or q.get("query"), "schema": schemas[q["db_id"]], "answer": text})
    _write_jsonl(args.out, rows)
    print(f"{len(rows)} candidates for {len(questions)} questions -> {args.out}")


def verify(args) -> None:
    rows = _read_jsonl(args.candidates)
    for r in rows:
        r["pred_sql"] = extract_sql(r["answer"])
        r["correct"] = is_correct(args.db_root, r["db_id"], r["pred_sql"], r["gold_sql"], args.timeout)
    _write_jsonl(args.out, rows)
    print(f"{sum(r['correct'] for r in rows)} of {len(rows)} candidates execute to the gold result")


def _group(rows: List[dict]) -> Dict[int, List[dict]]:
    g: Dict[int, List[dict]] = defaultdict(list)
    for r in rows:
        g[r["qid"]].append(r)
    return g


def sample_sft(rows: List[dict], per_question: int, seed: int) -> List[dict]:
    rng = random.Random(seed)
    out = []
    for qid, cands in sorted(_group(rows).items()):
        good = [c for c in cands if c["correct"]]
        rng.shuffle(good)
        for c in good[:per_question]:
            msgs = build_messages(c["schema"], c["question"], c["evidence"]) + [{"role": "assistant", "content": c["answer"]}]
            out.append({"messages": msgs})
    return out


def sample_dpo(rows: List[dict], per_question: int, seed: int) -> List[dict]:
    """Pairs (correct answer, incorrect answer) of the same question; questions with only one kind give no pair."""
    rng = random.Random(seed)
    out = []
    for qid, cands in sorted(_group(rows).items()):
        good = [c for c in cands if c["correct"]]
        bad = [c for c in cands if not c["correct"] and c.get("pred_sql")]
        rng.shuffle(good)
        rng.shuffle(bad)
        for g, b in list(zip(good, bad))[:per_question]:
            out.append({"prompt": build_messages(g["schema"], g["question"], g["evidence"]),
                        "chosen": g["answer"], "rejected": b["answer"]})
    return out


def _save_dataset(rows: List[dict], out_dir: str) -> None:
    from datasets import Dataset

    Dataset.from_list(rows).save_to_disk(out_dir)
    print(f"{len(rows)} rows -> {out_dir}")


def evaluate(args) -> None:
    rows = _read_jsonl(args.verified)
    groups = _group(rows)
    first = sum(c[0]["correct"] for c in groups.values())
    any_ok = sum(any(x["correct"] for x in c) for c in groups.values())
    print(json.dumps({"questions": len(groups), "execution_accuracy_first": first / max(1, len(groups)),
                      "pass_at_n": any_ok / max(1, len(groups))}))


def main() -> None:
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("generate")
    g.add_argument("--questions", required=True); g.add_argument("--schemas", required=True); g.add_argument("--out", required=True)
    g.add_argument("--model", required=True); g.add_argument("--n", type=int, default=8); g.add_argument("--temperature", type=float, default=0.8)
    g.add_argument("--client", choices=["vllm", "azure"], default="vllm"); g.add_argument("--work-dir", default="./excot_batches")
    g.add_argument("--credentials", default=None)
    v = sub.add_parser("verify")
    v.add_argument("--candidates", required=True); v.add_argument("--db-root", required=True); v.add_argument("--out", required=True)
    v.add_argument("--timeout", type=float, default=30.0)
    for name in ("sft", "dpo"):
        s = sub.add_parser(name)
        s.add_argument("--verified", required=True); s.add_argument("--out", required=True)
        s.add_argument("--per-question", type=int, default=1); s.add_argument("--seed", type=int, default=0)
    e = sub.add_parser("evaluate")
    e.add_argument("--verified", required=True)
    args = ap.parse_args()
    if args.cmd == "generate":
        generate(args)
    elif args.cmd == "verify":
        verify(args)
    elif args.cmd == "sft":
        _save_dataset(sample_sft(_read_jsonl(args.verified), args.per_question, args.seed), args.out)
    elif args.cmd == "dpo":
        _save_dataset(sample_dpo(_read_jsonl(args.verified), args.per_question, args.seed), args.out)
    else:
        evaluate(args)


if __name__ == "__main__":
    main()
