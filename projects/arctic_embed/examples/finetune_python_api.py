# SPDX-License-Identifier: Apache-2.0
"""Fine-tune a bi-encoder from Python instead of a YAML recipe: build the config dict, let `get_config` resolve it against
the trainer class, construct the trainer and call `train()`.  Run under the launcher (one process per GPU):

    python -m arctictraining_b200.launcher.local --num_gpus 8 -- python projects/arctic_embed/examples/finetune_python_api.py \
        --data data/train --model intfloat/e5-base-unsupervised

The reference shows the same usage in projects/arctic_embed/examples/finetune_models/finetune_e5_base_unsupervised.py.
"""

import argparse
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[3]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "projects" / "arctic_embed"))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--data", required=True, help="directory of batch_XXXXXXXX/ folders written by data_processing/pretokenize.py")
    ap.add_argument("--eval-data", default=None)
    ap.add_argument("--model", default="intfloat/e5-base-unsupervised")
    ap.add_argument("--out", default="./biencoder-ckpt")
    ap.add_argument("--lr", type=float, default=2e-5)
    ap.add_argument("--warmup-steps", type=int, default=100)
    ap.add_argument("--decay-steps", type=int, default=300)
    args = ap.parse_args()

    import train  # noqa: F401  registers the biencoder trainer, data factory and checkpoint engine

    from arctictraining_b200.config.trainer import get_config
    from arctictraining_b200.registry import get_registered_trainer

    recipe = {
        "type": "biencoder",
        "epochs": 1,
        "micro_batch_size": 1,
        "loss_temperature": 0.02,
        "mrl_dim": 256,
        "use_in_batch_negatives": True,
        "model": {"name_or_path": args.model, "pooling": "first", "attn_implementation": "sdpa"},
        "data": {"root_directory": args.data, "eval_root_directories": [args.eval_data] if args.eval_data else [],
                 "max_seq_length_query": 32, "max_seq_length_doc": 256},
        # ZeRO-1 with fp32 gradient reduction: contrastive gradients are small and every rank sees the whole batch
        "deepspeed": {"zero_optimization": {"stage": 1}, "communication_data_type": "fp32"},
        "optimizer": {"lr": args.lr, "weight_decay": 0.01},
        "scheduler": {"type": "wds", "num_warmup_steps": args.warmup_steps, "num_decay_steps": args.decay_steps},
        "checkpoint": [{"type": "biencoder", "output_dir": args.out, "save_end_of_training": True}],
        "logger": {"level": "INFO", "print_output_ranks": [0]},
    }
    config = get_config(recipe)
    trainer = get_registered_trainer(config.type)(config)
    trainer.train()


if __name__ == "__main__":
    main()
