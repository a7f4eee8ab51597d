# SPDX-License-Identifier: Apache-2.0
"""Write the job scripts of a data-generation run: for every dataset, `--num-shards` scripts that each run
`vllm_data_generation.py` on one shard.  `multigpu_runner.py <scripts dir>` then works through them.

    python make_datagen_jobs.py --model meta-llama/Llama-3.1-8B-Instruct --data-dir gen --scripts-dir gen_jobs \
        --datasets ultrachat magicoder --num-shards 8 --tensor-parallel 1 --temperature 0

Each script keeps vLLM's compile cache apart per GPU group (`VLLM_CACHE_ROOT`), because several replicas start at once.
Reference: projects/arctic_lstm_speculator/speculator/data_generation/data_gen_script_maker.py.
"""

from __future__ import annotations

import argparse
import os
import shlex
from typing import List
from typing import Optional
from typing import Sequence

_GENERATOR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "vllm_data_generation.py")


def job_script(model: str, dataset: str, shard: int, num_shards: int, out_path: str, tensor_parallel: int = 1,
               temperature: float = 1.0, tokenizer: Optional[str] = None, extra: Sequence[str] = ()) -> str:
    args = ["python", _GENERATOR, "--model", model, "--dataset", dataset, "--shard", str(shard), "--num-shards",
            str(num_shards), "--tensor-parallel", str(tensor_parallel), "--temperature", str(temperature), "--out",
            out_path]
    if tokenizer:
        args += ["--tokenizer", tokenizer]
    args += list(extra)
    return ("#!/usr/bin/env bash\nset -euo pipefail\n"
            "export VLLM_CACHE_ROOT=./vllm_cache/${CUDA_VISIBLE_DEVICES:-all}\n"
            + " ".join(shlex.quote(a) for a in args) + "\n")


def write_jobs(model: str, data_dir: str, scripts_dir: str, datasets: Sequence[str], num_shards: int,
               tensor_parallel: int = 1, temperature: float = 1.0, tokenizer: Optional[str] = None,
               prefix: str = "gen", extra: Sequence[str] = ()) -> List[str]:
    """Write `<scripts_dir>/<prefix>_<dataset>_<shard>.sh` for every (dataset, shard); returns the paths."""
    os.makedirs(scripts_dir, exist_ok=True)
    paths = []
    for dataset in datasets:
        tag = dataset.replace("/", "_").replace(":", "_")
        for shard in range(num_shards):
            out_path = os.path.join(data_dir, tag, f"{shard}_{num_shards}.jsonl")
            path = os.path.join(scripts_dir, f"{prefix}_{tag}_{shard:02d}.sh")
            with open(path, "w") as f:
                f.write(job_script(model, dataset, shard, num_shards, out_path, tensor_parallel, temperature,
                                   tokenizer, extra))
            paths.append(path)
    return paths


def main(argv: Optional[Sequence[str]] = None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--tokenizer", default=None)
    ap.add_argument("--data-dir", required=True, help="where the generated *.jsonl go")
    ap.add_argument("--scripts-dir", required=True)
    ap.add_argument("--datasets", nargs="+", default=["ultrachat", "magicoder"])
    ap.add_argument("--num-shards", type=int, default=8)
    ap.add_argument("--tensor-parallel", type=int, default=1)
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--prefix", default="gen")
    args, extra = ap.parse_known_args(argv)
    paths = write_jobs(args.model, args.data_dir, args.scripts_dir, args.datasets, args.num_shards,
                       args.tensor_parallel, args.temperature, args.tokenizer, args.prefix, extra)
    print(f"{len(paths)} job scripts -> {args.scripts_dir}")


if __name__ == "__main__":
    main()
