# SPDX-License-Identifier: Apache-2.0
"""Run a pre-tokenise-and-batch job from a config file (JSON or YAML).

    python projects/arctic_embed/data_processing/run_pretokenize_job.py pairs job.yaml [--num-shards 8 --shard 3]
    python projects/arctic_embed/data_processing/run_pretokenize_job.py mined job.yaml

``pairs`` validates the file as ``PairsJob`` (large-scale query/document pairs; shardable), ``mined`` as
``MinedDataJob`` (output of hard-negative mining).  Inputs and outputs may be local paths or ``s3://`` / ``gs://`` URLs.
"""

import sys

from arctictraining_b200.embed.data_processing import MinedDataJob
from arctictraining_b200.embed.data_processing import PairsJob
from arctictraining_b200.embed.data_processing import pretokenize_mined_data
from arctictraining_b200.embed.data_processing import pretokenize_pairs
from arctictraining_b200.embed.data_processing import run_config_file_cli

if __name__ == "__main__":
    kinds = {"pairs": (PairsJob, pretokenize_pairs), "mined": (MinedDataJob, pretokenize_mined_data)}
    if len(sys.argv) < 3 or sys.argv[1] not in kinds:
        sys.exit(__doc__)
    cls, job = kinds[sys.argv[1]]
    run_config_file_cli(cls, job, sys.argv[2:])
