# SPDX-License-Identifier: Apache-2.0
"""``python -m arctic_training_cli recipe.yaml --num_gpus N``: the module name under which the reference ships its
command line (arctic_training_cli.py:1-125); forwards to this package's CLI."""

import sys

from arctictraining_b200.cli import main

if __name__ == "__main__":
    sys.exit(main())
