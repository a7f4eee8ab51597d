# SPDX-License-Identifier: Apache-2.0
"""Generate speculator training data: let the base model continue real text with vLLM and store what it wrote.  A
speculator must imitate what the base model itself would write, so training on the model's own continuations beats
training on the human reference text.

Two ways to cut prompts out of a conversation dataset (`--prompt-mode`):

* `chunks` (default): render each conversation with the chat template, cut the token stream into consecutive pieces of
  `--prompt-tokens` tokens (the ragged tail is dropped) and let the model write `--gen-tokens` tokens after each piece
  with end-of-sequence ignored.  Every conversation yields many short prompts from all positions of a dialogue, and
  every continuation has the same length, so a training batch needs no padding.
* `turns`: one prompt per assistant turn - the conversation up to that turn plus the generation prompt.

Output: one JSON line per prompt, `{"input": [prompt ids], "output": [generated ids]}`.  One process per shard of the
dataset; run several (one per GPU group, see `make_datagen_jobs.py` and `multigpu_runner.py`) and merge with
`concat_generated_datasets.py`:

    python vllm_data_generation.py --model meta-llama/Llama-3.1-8B-Instruct --dataset ultrachat \
        --shard 0 --num-shards 8 --out gen/ultrachat/0_8.jsonl --tensor-parallel 1

`--dataset` is a short name (`ultrachat`, `magicoder`, `aya_<language>`) or `hub_path[:split]` of any dataset with a
`messages` column.  Reference: projects/arctic_lstm_speculator/speculator/data_generation/vllm_data_generation.py.
"""

from __future__ import annotations

import argparse
import json
import os
from typing import Any
from typing import Callable
from typing import Dict
from typing import Iterable
from typing import List
from typing import Tuple

# short name -> (hub path, config name or None, split, (question column, answer column) or None for `messages`)
KNOWN_DATASETS: Dict[str, Tuple[str, Any, str, Any]] = {
    "ultrachat": ("HuggingFaceH4/ultrachat_200k", None, "train_sft", None),
    "magicoder": ("ise-uiuc/Magicoder-OSS-Instruct-75K", None, "train", ("problem", "solution")),
}


def resolve_dataset(name: str) -> Tuple[str, Any, str, Any]:
    """(hub path, config, split, column pair) of a `--dataset` argument."""
    if name in KNOWN_DATASETS:
        return KNOWN_DATASETS[name]
    if name.startswith("aya_"):
        return ("CohereLabs/aya_collection_language_split", name[len("aya_"):], "test", ("inputs", "targets"))
    path, _, split = name.partition(":")
    return (path, None, split or "train", None)


def as_conversation(row: Dict[str, Any], columns) -> List[Dict[str, str]]:
    """The chat messages of one row; question / answer columns become a two-turn conversation."""
    if columns is None:
        return list(row["messages"])
    question, answer = columns
    return [{"role": "user", "content": row[question]}, {"role": "assistant", "content": row[answer]}]


def shard_range(n_rows: int, shard: int, num_shards: int) -> range:
    """Contiguous rows of shard `shard`; the shards tile `range(n_rows)` exactly."""
    if not 0 <= shard < num_shards:
        raise ValueError(f"shard {shard} is outside 0..{num_shards - 1}")
    return range(shard * n_rows // num_shards, (shard + 1) * n_rows // num_shards)


def chunk_prompts(token_ids: List[int], prompt_tokens: int) -> List[List[int]]:
    """Consecutive pieces of `prompt_tokens` tokens; a tail shorter than that is dropped."""
    whole = len(token_ids) // prompt_tokens * prompt_tokens
    return [list(token_ids[i:i + prompt_tokens]) for i in range(0, whole, prompt_tokens)]


def turn_prompts(messages: List[Dict[str, str]], tokenizer, max_prompt_tokens: int) -> List[List[int]]:
    """One prompt per assistant turn: the conversation before that turn, ending in the generation prompt."""
    prompts = []
    for i, m in enumerate(messages):
        if m["role"] != "assistant" or i == 0:
            continue
        ids = tokenizer.apply_chat_template(messages[:i], add_generation_prompt=True, tokenize=True)
        if len(ids) <= max_prompt_tokens:
            prompts.append(list(ids))
    return prompts


def build_prompts(conversations: Iterable[List[Dict[str, str]]], tokenizer, mode: str, prompt_tokens: int,
                  max_prompt_tokens: int) -> List[List[int]]:
    prompts: List[List[int]] = []
    for messages in conversations:
        if mode == "turns":
            prompts.extend(turn_prompts(messages, tokenizer, max_prompt_tokens))
        else:
            text = tokenizer.apply_chat_template(messages, tokenize=False)
            ids = tokenizer(text, add_special_tokens=False)["input_ids"]
            prompts.extend(chunk_prompts(list(ids), prompt_tokens))
    return prompts


def write_generations(path: str, prompts: List[List[int]], generate: Callable[[List[List[int]]], List[List[int]]],
                      batch: int = 4096) -> int:
    """Run `generate` over the prompts in batches and append one JSON line per prompt; a batch that was written
    survives a later crash.  Returns the number of lines written."""
    if os.path.dirname(path):
        os.makedirs(os.path.dirname(path), exist_ok=True)
    n = 0
    with open(path, "w") as f:
        for lo in range(0, len(prompts), batch):
            part = prompts[lo:lo + batch]
            for prompt, out in zip(part, generate(part)):
                f.write(json.dumps({"input": list(prompt), "output": list(out)}) + "\n")
                n += 1
            f.flush()
    return n


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--tokenizer", default=None)
    ap.add_argument("--dataset", default="ultrachat")
    ap.add_argument("--shard", type=int, default=0)
    ap.add_argument("--num-shards", type=int, default=1)
    ap.add_argument("--max-samples", type=int, default=0)
    ap.add_argument("--prompt-mode", choices=["chunks", "turns"], default="chunks")
    ap.add_argument("--prompt-tokens", type=int, default=64)
    ap.add_argument("--max-prompt-tokens", type=int, default=2048)
    ap.add_argument("--gen-tokens", type=int, default=256)
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--top-k", type=int, default=10)
    ap.add_argument("--tensor-parallel", type=int, default=1)
    ap.add_argument("--out", required=True)
    args = ap.parse_args()

    from datasets import load_dataset
    from transformers import AutoTokenizer
    from vllm import LLM
    from vllm import SamplingParams

    path, config, split, columns = resolve_dataset(args.dataset)
    data = load_dataset(path, config, split=split)
    rows = shard_range(len(data), args.shard, args.num_shards)
    if args.max_samples:
        rows = rows[:args.max_samples]
    data = data.select(rows)
    tok = AutoTokenizer.from_pretrained(args.tokenizer or args.model)
    prompts = build_prompts((as_conversation(r, columns) for r in data), tok, args.prompt_mode, args.prompt_tokens,
                            args.max_prompt_tokens)
    chunks = args.prompt_mode == "chunks"
    max_len = (args.prompt_tokens if chunks else args.max_prompt_tokens) + args.gen_tokens
    llm = LLM(model=args.model, tensor_parallel_size=args.tensor_parallel, max_model_len=max_len,
              enable_chunked_prefill=True, gpu_memory_utilization=0.9)
    sampling = SamplingParams(temperature=args.temperature, top_k=args.top_k if args.temperature > 0 else -1,
                              max_tokens=args.gen_tokens, ignore_eos=chunks, skip_special_tokens=False,
                              detokenize=False)

    def generate(part: List[List[int]]) -> List[List[int]]:
        outs = llm.generate([{"prompt_token_ids": p} for p in part], sampling)
        return [list(o.outputs[0].token_ids) for o in outs]

    n = write_generations(args.out, prompts, generate)
    print(f"{n} samples -> {args.out}")


if __name__ == "__main__":
    main()
