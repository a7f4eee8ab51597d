# SPDX-License-Identifier: Apache-2.0
"""Fetch what a recipe needs from the Hugging Face hub ahead of a run (CI caches, air-gapped clusters).

    python ci/prefetch_assets.py -c recipe.yaml -d data  [-t /scratch/tmp]
    python ci/prefetch_assets.py -c recipe.yaml -d model

``data`` loads every ``data.sources`` (and ``data.eval_sources``) entry once, which fills the datasets cache; ``model``
snapshots the weights, configuration and tokenizer of ``model.name_or_path`` (and ``tokenizer.name_or_path``).
Counterpart of scripts/download_data.py in the reference.
"""

import argparse
import os
import sys
import tempfile
from pathlib import Path
from typing import Any
from typing import Dict
from typing import Iterator
from typing import Tuple

import yaml


def iter_sources(config: Dict[str, Any]) -> Iterator[Tuple[str, Any, Dict[str, Any]]]:
    data = config.get("data", {}) or {}
    for key in ("sources", "eval_sources"):
        for src in data.get(key, []) or []:
            if isinstance(src, dict):
                path = src.get("name_or_path", src.get("type"))
                yield str(path), src.get("split"), dict(src.get("kwargs", {}) or {})
            else:
                yield str(src), None, {}


def model_ids(config: Dict[str, Any]):
    ids = [config.get("model", {}).get("name_or_path")]
    ids.append((config.get("tokenizer") or {}).get("name_or_path"))
    return [i for n, i in enumerate(ids) if i and i not in ids[:n]]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("-c", "--config", type=Path, required=True)
    ap.add_argument("-d", "--download", choices=["data", "model"], required=True)
    ap.add_argument("-t", "--tmp-path", type=Path, default=Path(tempfile.gettempdir()))
    ap.add_argument("--list", action="store_true", help="print what would be fetched and exit")
    args = ap.parse_args(argv)
    config = yaml.safe_load(args.config.read_text())
    if args.download == "data":
        os.makedirs(args.tmp_path, exist_ok=True)
        tempfile.tempdir = str(args.tmp_path)
        for path, split, kwargs in iter_sources(config):
            print(f"dataset {path} split={split} kwargs={kwargs}")
            if not args.list and not os.path.exists(path):
                from datasets import load_dataset

                load_dataset(path=path, split=split, **kwargs)
    else:
        for name in model_ids(config):
            print(f"model {name}")
            if not args.list and not os.path.isdir(name):
                from huggingface_hub import snapshot_download

                snapshot_download(name)
    return 0


if __name__ == "__main__":
    sys.exit(main())
