# SPDX-License-Identifier: Apache-2.0
"""Generate base-model continuations with several `vllm serve` replicas (one per GPU group) and store them as a
pre-tokenised Hugging Face dataset for speculator training.  Uses `MultiReplicaVllmSynth`, which starts the servers,
waits until they answer, fans the requests out over them and stops them again.

    python vllm_multi_replica_gen.py --model meta-llama/Llama-3.1-8B-Instruct --dataset HuggingFaceH4/ultrachat_200k \
        --split train_sft --replicas 8 --tensor-parallel 1 --max-samples 20000 --out gen/ultrachat

Reference: projects/mlp_speculator/mlp_speculator/data_generation/vllm_multi_replica_gen_hf_datasets.py.
"""

import argparse


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--dataset", required=True)
    ap.add_argument("--split", default="train")
    ap.add_argument("--replicas", type=int, default=8)
    ap.add_argument("--tensor-parallel", type=int, default=1)
    ap.add_argument("--max-samples", type=int, default=0)
    ap.add_argument("--gen-tokens", type=int, default=256)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--out", required=True)
    args = ap.parse_args()

    from datasets import Dataset
    from datasets import load_dataset
    from transformers import AutoTokenizer

    from arctictraining_b200.synth import MultiReplicaVllmSynth

    tok = AutoTokenizer.from_pretrained(args.model)
    data = load_dataset(args.dataset, split=args.split)
    if args.max_samples:
        data = data.select(range(min(args.max_samples, len(data))))
    client = MultiReplicaVllmSynth(
        model=args.model, n_replicas=args.replicas, tensor_parallel=args.tensor_parallel,
        sampling={"temperature": args.temperature, "max_tokens": args.gen_tokens},
    )
    prompts = {}
    for row in data:
        msgs = row.get("messages") or []
        for i, m in enumerate(msgs):
            if m["role"] == "assistant" and i > 0:
                cid = client.add_chat_to_batch_task("gen", messages=msgs[:i])
                prompts[cid] = msgs[:i]
    try:
        outputs = client.extract_messages_from_responses(client.execute_batch_task("gen"))
    finally:
        client.teardown()
    rows = []
    lost = 0
    for o in outputs:
        if not o["choices"]:  # the request failed on every replica it was tried on
            lost += 1
            continue
        prompt_ids = tok.apply_chat_template(prompts[o["custom_id"]], add_generation_prompt=True, tokenize=True)
        gen_ids = tok(o["choices"][0]["content"], add_special_tokens=False)["input_ids"]
        rows.append({"input_ids": prompt_ids + gen_ids, "labels": [-100] * len(prompt_ids) + gen_ids})
    Dataset.from_list(rows).save_to_disk(args.out)
    print(f"{len(rows)} samples -> {args.out} ({lost} requests lost)")


if __name__ == "__main__":
    main()
