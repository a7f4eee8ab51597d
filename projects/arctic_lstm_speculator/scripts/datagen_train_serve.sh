#!/usr/bin/env bash
# SPDX-License-Identifier: Apache-2.0
# Data generation -> speculator training -> serving with speculative decoding, for one base model on one 8-GPU node.
#
#   bash datagen_train_serve.sh <base model> <recipe.yaml> [vllm tensor-parallel size for generation]
#   bash datagen_train_serve.sh meta-llama/Llama-3.1-8B-Instruct ../llama3.1-8b.yaml 1
#   bash datagen_train_serve.sh meta-llama/Llama-3.3-70B-Instruct ../llama3.3-70b.yaml 4
#   bash datagen_train_serve.sh openai/gpt-oss-120b ../oss-120b.yaml 8
#
# Switches (environment): DATA_GEN=0 skips generation, TRAIN=0 skips training, SERVE=0 skips serving;
# GEN_DIR (generated data), NUM_SHARDS (job scripts per dataset), DATASETS, GEN_TEMP, NUM_SPEC_TOKENS.
# The recipe must read "$GEN_DIR/all" (`type: huggingface`, `process: false`) and write its checkpoint to SPEC_DIR.
set -euo pipefail
MODEL=${1:?base model}
RECIPE=${2:?recipe yaml}
TP=${3:-1}
HERE=$(cd "$(dirname "$0")/.." && pwd)
GEN=${GEN_DIR:-$HERE/gen}
SPEC=${SPEC_DIR:-$HERE/spec-ckpt}
DATASETS=${DATASETS:-"ultrachat magicoder"}

if [ "${DATA_GEN:-1}" -eq 1 ]; then
  # shellcheck disable=SC2086
  python "$HERE/data_generation/make_datagen_jobs.py" --model "$MODEL" --data-dir "$GEN/raw" \
      --scripts-dir "$GEN/jobs" --datasets $DATASETS --num-shards "${NUM_SHARDS:-16}" --tensor-parallel "$TP" \
      --temperature "${GEN_TEMP:-0}"
  python "$HERE/data_generation/multigpu_runner.py" "$GEN/jobs" --max-gpus 8 -n "$TP"
  python "$HERE/data_generation/concat_generated_datasets.py" --inputs "$GEN/raw" --out "$GEN/all"
fi

if [ "${TRAIN:-1}" -eq 1 ]; then
  arctic_training "$RECIPE" --num_gpus 8
fi

if [ "${SERVE:-1}" -eq 1 ]; then
  vllm serve "$MODEL" --tensor-parallel-size 8 --enable-chunked-prefill --gpu-memory-utilization 0.9 \
      --speculative-config "{\"model\": \"$SPEC\", \"num_speculative_tokens\": ${NUM_SPEC_TOKENS:-3}, \"draft_tensor_parallel_size\": 8, \"method\": \"arctic\"}"
fi
