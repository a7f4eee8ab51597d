#!/usr/bin/env bash
# SPDX-License-Identifier: Apache-2.0
# Data generation -> speculator training -> serving with speculative decoding, for one base model on one 8-GPU node.
# Usage: bash datagen_train_serve.sh meta-llama/Llama-3.1-8B-Instruct
set -euo pipefail
MODEL=${1:?base model}
HERE=$(cd "$(dirname "$0")/.." && pwd)
GEN=${GEN_DIR:-$HERE/gen}

# 1. base-model continuations, one shard per GPU
: > "$GEN.jobs"
for s in $(seq 0 7); do
  echo "python $HERE/data_generation/vllm_data_generation.py --model $MODEL --dataset HuggingFaceH4/ultrachat_200k --split train_sft --shard $s --num-shards 8 --out $GEN/shard$s" >> "$GEN.jobs"
done
python "$HERE/data_generation/multigpu_runner.py" --commands "$GEN.jobs" --gpus-per-job 1
python "$HERE/data_generation/concat_generated_datasets.py" --inputs "$GEN"/shard* --out "$GEN/all"

# 2. train the speculator heads on the frozen base model (the recipe reads $GEN/all with `process: false`)
arctic_training "$HERE/llama3.1-8b.yaml" --num_gpus 8

# 3. serve the base model with the trained speculator
vllm serve "$MODEL" --speculative-config "{\"model\": \"$HERE/spec-ckpt\", \"num_speculative_tokens\": 3}"
