# SPDX-License-Identifier: Apache-2.0
"""Evaluate every checkpoint of a training run: sample with ``infer.py``, score with ``evaluate_bird.py``, collect the
accuracies per checkpoint in one JSON file (and a plot when matplotlib is available).

    python projects/arctic_text2sql_r1/auto_evaluation.py --ckpt-dir out/ --input dev_bird.json --gold dev.json \\
        --db_path dev_databases --n 8 --out-dir eval_results

Parity: projects/arctic_text2sql_r1/bird_eval/auto_evaluation.py.
"""

import argparse
import json
import re
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))

from text2sql.evaluate import load_json  # noqa: E402
from text2sql.evaluate import run_eval  # noqa: E402


def checkpoints(ckpt_dir: str):
    """``global_step_<N>`` sub-directories in step order (a directory that holds a model itself counts as one)."""
    root = Path(ckpt_dir)
    steps = sorted((int(m.group(1)), p) for p in root.iterdir() if p.is_dir() and (m := re.match(r"global_step_?(\d+)$", p.name)))
    return steps or [(0, root)]


def plot(acc: dict, path: Path) -> bool:
    try:
        import matplotlib

        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except ImportError:
        return False
    for mode, series in acc.items():
        xs = sorted(series, key=int)
        plt.plot([int(x) for x in xs], [series[x] for x in xs], marker="o", label=mode)
    plt.xlabel("step")
    plt.ylabel("execution accuracy")
    plt.legend()
    plt.savefig(path)
    return True


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ckpt-dir", required=True)
    ap.add_argument("--input", required=True)
    ap.add_argument("--gold", required=True)
    ap.add_argument("--db_path", required=True)
    ap.add_argument("--n", type=int, default=8)
    ap.add_argument("--temperature", type=float, default=0.8)
    ap.add_argument("--tensor-parallel-size", type=int, default=1)
    ap.add_argument("--out-dir", default="eval_results")
    args = ap.parse_args()
    out = Path(args.out_dir)
    out.mkdir(parents=True, exist_ok=True)
    gold = load_json(args.gold)
    acc = {"greedy_search": {}, "major_voting": {}, "pass@k": {}}
    for step, path in checkpoints(args.ckpt_dir):
        pred = out / f"pred_step_{step}.json"
        if not pred.exists():
            subprocess.run([sys.executable, str(HERE / "infer.py"), "--model", str(path), "--input", args.input, "--output", str(pred),
                            "--n", str(args.n), "--temperature", str(args.temperature),
                            "--tensor-parallel-size", str(args.tensor_parallel_size)], check=True)
        preds = load_json(str(pred))
        for mode in acc:
            acc[mode][str(step)] = run_eval(gold, preds, args.db_path, mode)[0]
        (out / "accuracy.json").write_text(json.dumps(acc, indent=2))
    plot(acc, out / "accuracy.png")
    print(json.dumps(acc))


if __name__ == "__main__":
    main()
