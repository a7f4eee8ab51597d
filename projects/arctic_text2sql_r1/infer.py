# SPDX-License-Identifier: Apache-2.0
"""Sample answers for prepared inputs with vLLM and keep the SQL of every sample.

    python projects/arctic_text2sql_r1/infer.py --model <path> --input dev_bird.json --output preds.json --n 8 \\
        --temperature 0.8 [--tensor-parallel-size 4]

Output: the input rows with ``responses`` (texts) and ``pred_sqls`` (the last ```sql block of each) added.
Parity: projects/arctic_text2sql_r1/bird_eval/infer.py.
"""

import argparse
import json
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))

from text2sql.evaluate import load_json  # noqa: E402
from text2sql.evaluate import parse_response  # noqa: E402


def attach_predictions(rows, responses_per_row):
    out = []
    for row, texts in zip(rows, responses_per_row):
        out.append({**row, "responses": list(texts), "pred_sqls": [parse_response(t) for t in texts]})
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--input", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--n", type=int, default=1)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--max-tokens", type=int, default=4096)
    ap.add_argument("--tensor-parallel-size", type=int, default=1)
    args = ap.parse_args()

    from vllm import LLM
    from vllm import SamplingParams

    rows = load_json(args.input)
    llm = LLM(model=args.model, tensor_parallel_size=args.tensor_parallel_size, dtype="bfloat16")
    tok = llm.get_tokenizer()
    prompts = [tok.apply_chat_template([{"role": "user", "content": r["input_seq"]}], add_generation_prompt=True, tokenize=False)
               for r in rows]
    params = SamplingParams(n=args.n, temperature=args.temperature if args.n > 1 or args.temperature else 0.0,
                            max_tokens=args.max_tokens)
    outs = llm.generate(prompts, params)
    result = attach_predictions(rows, [[c.text for c in o.outputs] for o in outs])
    Path(args.output).write_text(json.dumps(result, indent=2, ensure_ascii=False))
    print(f"wrote {len(result)} rows with {args.n} samples each to {args.output}")


if __name__ == "__main__":
    main()
