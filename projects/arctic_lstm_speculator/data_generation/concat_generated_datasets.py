# SPDX-License-Identifier: Apache-2.0
"""Merge the per-shard outputs of `vllm_data_generation.py` into one dataset directory.

    python concat_generated_datasets.py --inputs gen/shard* --out gen/all
"""

import argparse


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--inputs", nargs="+", required=True)
    ap.add_argument("--out", required=True)
    args = ap.parse_args()
    from datasets import concatenate_datasets
    from datasets import load_from_disk

    merged = concatenate_datasets([load_from_disk(p) for p in sorted(args.inputs)])
    merged.save_to_disk(args.out)
    print(f"{len(merged)} samples -> {args.out}")


if __name__ == "__main__":
    main()
