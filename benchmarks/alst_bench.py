# SPDX-License-Identifier: Apache-2.0
"""Long-sequence (ALST) SFT step time: one synthetic sequence of ``--seq-len`` tokens per step, Ulysses sequence
parallelism over all ranks, tiled MLP, tiled fused cross-entropy, activation checkpointing (optionally with host
offload), ZeRO-3 bf16.  Timed on the device (CUDA events, max over ranks) through the trainer's public ``step``.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29533 \
        benchmarks/alst_bench.py --seq-len 131072 --steps 2 --warmup 1

Reference recipes with the same switches: projects/sequence-parallelism/run-h100-sp8-llama-8b.yml:1-60.
"""

import argparse
import json
import os
import sys
import tempfile
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama-3.1-8b")
    ap.add_argument("--seq-len", type=int, default=131072, help="tokens of the whole sequence (all ranks together)")
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--attn", default="native")
    ap.add_argument("--no-tiled-mlp", action="store_true")
    ap.add_argument("--act-offload", action="store_true", help="checkpointed activations go to pinned host memory")
    ap.add_argument("--keep", default="auto")
    ap.add_argument("--fused-comm", default="auto", choices=["auto", "off"])
    ap.add_argument("--optimizer", default="fused_adam", choices=["fused_adam", "cpu_adam"],
                    help="cpu_adam: optimizer states in pinned host memory (zero_optimization.offload_optimizer)")
    ap.add_argument("--offload-ratio", type=float, default=1.0, help="fraction of the optimizer states kept on the host")
    ap.add_argument("--offload-param", action="store_true", help="parameter shards in pinned host memory too")
    ap.add_argument("--bf16-optimizer", action="store_true",
                    help="bf16 master weights, gradients and AdamW moments (6 bytes per parameter instead of 16)")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("AT_LOG_LEVEL", "WARNING")
    os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")
    if args.fused_comm == "off":
        os.environ["ATB200_FUSED_COMM"] = "0"

    from arctictraining_b200 import ops
    from arctictraining_b200.comm.dist import init_distributed
    from arctictraining_b200.config.trainer import get_config
    from arctictraining_b200.ops import _ext
    from arctictraining_b200.parallel.ulysses import shard_batch_for_rank
    from arctictraining_b200.registry import get_registered_trainer

    init_distributed(local_rank)
    _ext.require()
    device = torch.device("cuda", torch.cuda.current_device())
    S = args.seq_len
    assert S % (world * 128) == 0, "sequence length must be a multiple of 128 x ranks"

    workdir = Path(tempfile.gettempdir()) / f"atb200_alst_{os.getuid()}"
    zero = {"stage": 3}
    if args.optimizer == "cpu_adam":
        zero["offload_optimizer"] = {"device": "cpu", "ratio": args.offload_ratio}
    if args.offload_param:
        zero["offload_param"] = {"device": "cpu"}
    recipe = {
        "type": "sft",
        "micro_batch_size": 1,
        "epochs": 1,
        "seed": 42,
        "sequence_parallel_size": world,
        "tiled_mlp_compute": not args.no_tiled_mlp,
        "activation_checkpoint_cpu_offload": args.act_offload,
        "model": {"name_or_path": args.model, "dtype": "bf16", "attn_implementation": args.attn,
                  "hf_config_kwargs": {"num_hidden_layers": args.layers} if args.layers else {}},
        "data": {"sources": [{"type": "synthetic", "num_samples": 8 * world, "min_length": 64, "max_length": 128}],
                 "cache_dir": str(workdir / "cache"), "max_length": 128, "dl_num_workers": 0, "num_proc": 1},
        "optimizer": {"type": args.optimizer, "lr": 1e-5, "weight_decay": 0.1},
        "scheduler": {"name": "constant"},
        "deepspeed": {"zero_optimization": zero, "gradient_clipping": 1.0, "activation_checkpoint_keep": args.keep,
                      **({"bf16": {"enabled": True, "bf16_master_weights_and_grads": True, "bf16_optimizer_states": True}}
                         if args.bf16_optimizer else {})},
        "train_log_iter_interval": 0,
        "train_log_metrics_path": str(workdir / f"metrics_{rank}.jsonl"),
        "logger": {"level": "WARNING"},
    }
    trainer = get_registered_trainer("sft")(get_config(recipe))
    vocab = trainer.model.module.config["vocab_size"]

    def make_batch(seed: int):
        g = torch.Generator().manual_seed(seed)
        ids = torch.randint(8, vocab, (1, S), generator=g)
        labels = ids.clone()
        labels[:, : S // 2] = -100
        full = {"input_ids": ids, "labels": labels, "position_ids": torch.arange(S)[None]}
        local = shard_batch_for_rank(full, trainer.sp_rank if world > 1 else 0, world) if world > 1 else full
        return {k: (v.pin_memory() if torch.is_tensor(v) else v) for k, v in local.items()}

    def sync():
        if world > 1:
            dist.barrier(device_ids=[device.index])
        torch.cuda.synchronize()

    def do_step(b):
        if trainer.metrics.enabled:
            trainer.metrics.values.clear()
        trainer.step(b)  # H2D of the pinned batch, forward, backward, optimizer step, loss read-back

    for i in range(args.warmup):
        do_step(make_batch(i))
    sync()
    torch.cuda.reset_peak_memory_stats()
    batches = [make_batch(100 + i) for i in range(args.steps)]
    launches0 = ops.LAUNCH_COUNTER["native"]
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for b in batches:
        do_step(b)
    end.record()
    sync()
    ms = torch.tensor([start.elapsed_time(end)], device=device, dtype=torch.float64)
    mem = torch.tensor([torch.cuda.max_memory_allocated() / 2**30], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(mem, op=dist.ReduceOp.MAX)
    err = int(torch.ops.atb200.read_and_clear_error_flag(torch.zeros(1, device=device)))
    if trainer.config.sequence_parallel_size > 1 and trainer.sp_context._peer is not None:
        trainer.sp_context._peer.symm.check()
    if rank == 0:
        s_per_iter = float(ms) / 1e3 / args.steps
        eng = trainer.model
        res = {
            "metric": "alst_seconds_per_iteration", "value": round(s_per_iter, 3), "unit": "s/iter",
            "tokens_per_s": round(S / s_per_iter, 1), "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "config": {"model": args.model, "layers": eng.module.config["num_hidden_layers"], "seq_len": S,
                       "parallelism": f"ulysses-sp{world} + zero3", "tiled_mlp": not args.no_tiled_mlp,
                       "tiled_cross_entropy": True, "activation_offload": args.act_offload, "attention": args.attn,
                       "peer_memory_exchange": bool(world > 1 and trainer.sp_context.fused),
                       "attention_blocks_with_exchange_in_gemm": trainer.sp_context.fused_block_calls if world > 1 else 0,
                       "layers_keeping_activations": eng._keep_state.get("kept_layers", 0),
                       "optimizer": args.optimizer, "offload_optimizer_ratio": args.offload_ratio if args.optimizer == "cpu_adam" else 0.0,
                       "offload_param": args.offload_param, "bf16_optimizer_states": args.bf16_optimizer,
                       "attention_backward": os.getenv("ATB200_ATTN_BWD", "native")},
            "max_memory_gib_per_gpu": round(float(mem), 2), "gpu_launches": ops.LAUNCH_COUNTER["native"] - launches0,
            "kernel_error_flag": err,
        }
        print(json.dumps(res))
        if args.out:
            with open(args.out, "a") as f:
                f.write(json.dumps(res) + "\n")
    if world > 1:
        dist.barrier(device_ids=[device.index])
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
