# SPDX-License-Identifier: Apache-2.0
"""``arctic_training`` command line.  Parity: arctic_training_cli.py:24-125.

``arctic_training [train|process-data] recipe.yaml [--python_profile ...] [--launcher local|deepspeed|ray]
<launcher args>``: unknown arguments go to the process launcher (``--num_gpus 8 --master_port 29501`` ...).
``deepspeed`` is accepted as an alias of the built-in launcher so existing command lines keep working.
"""

from __future__ import annotations

import argparse
import os
import sys
from pathlib import Path
from typing import List
from typing import Optional


def local_launch(config_file: str, mode: str, python_profile: str, launcher_args: List[str]) -> int:
    from .launcher.local import main as launch_main

    worker = [sys.executable, "-u", "-m", "arctictraining_b200.entrypoint", "--mode", mode, "--config", config_file,
              "--python_profile", python_profile]
    return launch_main([*launcher_args, "--", *worker])


def ray_launch(config_file: str, mode: str, python_profile: str) -> None:
    from .launcher.ray_launcher import launch

    launch(config_file=config_file, mode=mode, python_profile=python_profile)


def main(argv: Optional[List[str]] = None) -> int:
    parser = argparse.ArgumentParser(
        prog="arctic_training",
        description="Launch a training recipe. Arguments after the recipe path are passed to the process launcher, "
                    "e.g. `arctic_training recipe.yaml --num_gpus 8`.",
    )
    parser.add_argument("mode", type=str, nargs="?", choices=["train", "process-data"], default="train")
    parser.add_argument("config", type=Path, help="Recipe YAML file.")
    parser.add_argument("--python_profile", type=str, choices=["tottime", "cumtime", "disable"], default="disable")
    parser.add_argument("--launcher", type=str, choices=["local", "deepspeed", "ray"], default=None)
    args, launcher_args = parser.parse_known_args(argv)
    if not args.config.exists():
        raise FileNotFoundError(f"Config file {args.config} not found.")
    use_ray = args.launcher == "ray" or (args.launcher is None and os.environ.get("USE_RAY", "").lower() in ("1", "true"))
    if use_ray:
        if launcher_args:
            raise ValueError("Process-launcher arguments are not supported with the Ray launcher.")
        ray_launch(str(args.config), args.mode, args.python_profile)
        return 0
    return local_launch(str(args.config), args.mode, args.python_profile, launcher_args)


if __name__ == "__main__":
    sys.exit(main())
