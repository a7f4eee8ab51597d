# SPDX-License-Identifier: Apache-2.0
"""Merge the `*.jsonl` files that `vllm_data_generation.py` wrote (searched recursively under `--inputs`) into one
Hugging Face dataset with pre-tokenised `input_ids` / `labels`, which a recipe reads with `process: false`:

    python concat_generated_datasets.py --inputs gen --out gen/all [--with-prompt]

By default a sample is the generated continuation alone (`input_ids == labels`): the speculator learns the model's own
text.  `--with-prompt` keeps the prompt in front with its labels masked (-100).
Reference: projects/arctic_lstm_speculator/speculator/data_generation/concat_generated_datasets.py.
"""

from __future__ import annotations

import argparse
import glob
import json
import os
from typing import Dict
from typing import Iterable
from typing import List


def find_generation_files(roots: Iterable[str]) -> List[str]:
    files: List[str] = []
    for root in roots:
        if os.path.isdir(root):
            files.extend(glob.glob(os.path.join(root, "**", "*.jsonl"), recursive=True))
        elif os.path.exists(root):
            files.append(root)
    return sorted(set(files))


def read_generations(files: Iterable[str], with_prompt: bool = False) -> Dict[str, List[List[int]]]:
    """Columns `input_ids` / `labels` of all lines of `files`; a truncated last line (a killed writer) is skipped."""
    input_ids: List[List[int]] = []
    labels: List[List[int]] = []
    for path in files:
        with open(path) as f:
            for line in f:
                line = line.strip()
                if not line:
                    continue
                try:
                    row = json.loads(line)
                except json.JSONDecodeError:
                    continue
                prompt, out = list(row.get("input", [])), list(row["output"])
                if not out:
                    continue
                if with_prompt:
                    input_ids.append(prompt + out)
                    labels.append([-100] * len(prompt) + out)
                else:
                    input_ids.append(out)
                    labels.append(out)
    return {"input_ids": input_ids, "labels": labels}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--inputs", nargs="+", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--with-prompt", action="store_true")
    args = ap.parse_args()
    from datasets import Dataset

    files = find_generation_files(args.inputs)
    if not files:
        raise SystemExit(f"no *.jsonl under {args.inputs}")
    merged = Dataset.from_dict(read_generations(files, args.with_prompt))
    merged.save_to_disk(args.out)
    print(f"{len(merged)} samples from {len(files)} files -> {args.out}")


if __name__ == "__main__":
    main()
