# SPDX-License-Identifier: Apache-2.0
"""Evaluate a SwiftKV checkpoint with lm-evaluation-harness.  The harness builds models through
`transformers.AutoModelForCausalLM`; a SwiftKV export is a plain checkpoint directory whose `config.json` carries the
SwiftKV fields, so this wrapper loads it with this package's model class and hands the module to the harness.

    python projects/swiftkv/eval.py --checkpoint /path/to/export --tasks arc_challenge,hellaswag --batch-size 8

The reference does the same by registering its model classes before calling the harness CLI (projects/swiftkv/eval.py).
"""

import argparse
import json
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent.parent))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--checkpoint", required=True)
    ap.add_argument("--tasks", default="arc_challenge")
    ap.add_argument("--batch-size", type=int, default=8)
    ap.add_argument("--limit", type=int, default=None)
    args = ap.parse_args()
    try:
        import lm_eval
        from lm_eval.models.huggingface import HFLM
    except ImportError as e:  # pragma: no cover - optional dependency
        raise SystemExit("lm-eval is not installed (pip install lm-eval)") from e
    import torch
    from transformers import AutoTokenizer

    sys.path.insert(0, str(Path(__file__).resolve().parent))
    from train import build_swiftkv_model  # the student model with shared-KV layers

    model = build_swiftkv_model(args.checkpoint, dtype=torch.bfloat16, device="cuda").eval()
    lm = HFLM(pretrained=model, tokenizer=AutoTokenizer.from_pretrained(args.checkpoint), batch_size=args.batch_size)
    results = lm_eval.simple_evaluate(model=lm, tasks=args.tasks.split(","), limit=args.limit)
    print(json.dumps(results["results"], indent=2, default=str))


if __name__ == "__main__":
    main()
