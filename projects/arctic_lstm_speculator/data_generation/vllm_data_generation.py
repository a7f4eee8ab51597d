# SPDX-License-Identifier: Apache-2.0
"""Generate speculator training data: let the base model continue real prompts with vLLM and store prompt + continuation
as pre-tokenised `input_ids` / `labels` (a Hugging Face dataset consumed with `process: false`, see
projects/arctic_lstm_speculator/llama3.1-8b.yaml).  A speculator must imitate what the base model itself would write,
so training on the model's own continuations beats training on the human reference text.

One process per dataset shard; run several (one per GPU group) and merge with `concat_generated_datasets.py`:

    python vllm_data_generation.py --model meta-llama/Llama-3.1-8B-Instruct --dataset HuggingFaceH4/ultrachat_200k \
        --split train_sft --shard 0 --num-shards 8 --out gen/shard0 --tensor-parallel 1

Reference: projects/arctic_lstm_speculator/speculator/data_generation/vllm_data_generation.py.
"""

from __future__ import annotations

import argparse
from typing import List


def conversation_prompts(row: dict, tokenizer, max_prompt_tokens: int) -> List[List[int]]:
    """One prompt per assistant turn: the conversation up to (not including) that turn, with the generation prompt."""
    msgs = row.get("messages") or []
    prompts = []
    for i, m in enumerate(msgs):
        if m["role"] != "assistant" or i == 0:
            continue
        ids = tokenizer.apply_chat_template(msgs[:i], add_generation_prompt=True, tokenize=True)
        if len(ids) <= max_prompt_tokens:
            prompts.append(ids)
    return prompts


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--dataset", required=True)
    ap.add_argument("--split", default="train")
    ap.add_argument("--shard", type=int, default=0)
    ap.add_argument("--num-shards", type=int, default=1)
    ap.add_argument("--max-samples", type=int, default=0)
    ap.add_argument("--max-prompt-tokens", type=int, default=2048)
    ap.add_argument("--gen-tokens", type=int, default=256)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--tensor-parallel", type=int, default=1)
    ap.add_argument("--out", required=True)
    args = ap.parse_args()

    from datasets import Dataset
    from datasets import load_dataset
    from transformers import AutoTokenizer
    from vllm import LLM
    from vllm import SamplingParams

    tok = AutoTokenizer.from_pretrained(args.model)
    data = load_dataset(args.dataset, split=args.split).shard(num_shards=args.num_shards, index=args.shard)
    if args.max_samples:
        data = data.select(range(min(args.max_samples, len(data))))
    prompts: List[List[int]] = []
    for row in data:
        prompts.extend(conversation_prompts(row, tok, args.max_prompt_tokens))
    llm = LLM(model=args.model, tensor_parallel_size=args.tensor_parallel)
    outs = llm.generate([{"prompt_token_ids": p} for p in prompts],
                        SamplingParams(temperature=args.temperature, max_tokens=args.gen_tokens))
    rows = []
    for p, o in zip(prompts, outs):
        gen = list(o.outputs[0].token_ids)
        rows.append({"input_ids": p + gen, "labels": [-100] * len(p) + gen})
    Dataset.from_list(rows).save_to_disk(args.out)
    print(f"{len(rows)} samples -> {args.out}")


if __name__ == "__main__":
    main()
