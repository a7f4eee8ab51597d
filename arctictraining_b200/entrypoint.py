# SPDX-License-Identifier: Apache-2.0
"""Per-rank entry point (``arctic_training_run``).  Parity: arctic_training/entrypoint.py:27-83."""

from __future__ import annotations

import argparse
import os
from pathlib import Path

import torch.distributed as dist

from .config.trainer import get_config
from .registry import get_registered_trainer


def launch(argv=None) -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--mode", type=str, choices=["train", "process-data"], default="train",
                        help="'process-data' only runs the data pipeline (fills the cache).")
    parser.add_argument("--config", type=Path, required=True, help="Recipe to run.")
    parser.add_argument("--local_rank", type=int, default=int(os.getenv("LOCAL_RANK", 0)))
    parser.add_argument("--python_profile", type=str, choices=["tottime", "cumtime", "disable"], default="disable",
                        help="Run training under cProfile on local rank 0, sorted by this key.")
    args = parser.parse_args(argv)
    if not args.config.exists():
        raise FileNotFoundError(f"Config file {args.config} not found.")
    os.environ.setdefault("LOCAL_RANK", str(args.local_rank))

    config = get_config(args.config)
    trainer = get_registered_trainer(name=config.type)(config, mode=args.mode)
    if args.mode == "train":
        if args.python_profile == "disable" or args.local_rank != 0:
            trainer.train()
        else:
            import cProfile
            from pstats import SortKey

            key = SortKey.TIME if args.python_profile == "tottime" else SortKey.CUMULATIVE
            cProfile.runctx("trainer.train()", None, {"trainer": trainer}, sort=key)
    if dist.is_initialized():
        try:
            dist.barrier()
        finally:
            dist.destroy_process_group()


if __name__ == "__main__":
    launch()
