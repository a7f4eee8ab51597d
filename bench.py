#!/usr/bin/env python
# SPDX-License-Identifier: Apache-2.0
"""Headline benchmark: Llama-3.1-8B supervised fine-tuning throughput (tokens/s) on N B200 GPUs.

Config (the one the baseline names): Llama-3.1-8B architecture, random-init bf16 weights, ZeRO-3, AdamW with
fp32 master weights, sequence length 8192 packed from variable-length synthetic samples (lengths uniform in
[256, 4096]), micro-batch 1 per GPU, activation checkpointing.  One step = forward + backward + optimizer
step.  ``value`` is device-timed (CUDA events, max over ranks) with inputs already on the device; ``e2e`` runs
the same steps through the public trainer API (``SFTTrainer.step``) including the host->device copy of each
batch from pinned memory and the device->host read of the loss.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        bench.py --gpus 8 --steps 5 --warmup 3
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "llama3.1_8b_sft_tokens_per_s"


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=5)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", type=str, default="native", choices=["native", "reference", "library_stack"],
                   help="native: this framework; reference: the unmodified reference (unavailable offline); library_stack: "
                        "a stand-in built from stock libraries (transformers + flash-attn + Liger + FSDP2), never "
                        "labelled as the reference")
    p.add_argument("--library-attn", type=str, default="flash_attention_2", help="attn_implementation of the library stack")
    p.add_argument("--no-liger", action="store_true", help="library stack without the Liger kernels")
    p.add_argument("--no-grad-ckpt", action="store_true", help="library stack without gradient checkpointing")
    p.add_argument("--model", type=str, default="llama-3.1-8b")
    p.add_argument("--seq-len", type=int, default=8192)
    p.add_argument("--zero-stage", type=int, default=3)
    p.add_argument("--layers", type=int, default=0, help="override the number of layers (debugging only; marks the result invalid)")
    p.add_argument("--attn", type=str, default="native")
    p.add_argument("--keep", type=str, default="auto",
                   help="layers that keep activations instead of recomputing them: a count, or auto (by free memory)")
    p.add_argument("--gemm", type=str, default=os.getenv("ATB200_GEMM", "tcgen05"), choices=["tcgen05", "cublas"])
    p.add_argument("--skip-e2e", action="store_true")
    p.add_argument("--torch-profile", type=str, default=None,
                   help="write a torch.profiler kernel table of the timed steps of rank 0 to this file (the number "
                        "printed by such a run is not a benchmark value)")
    p.add_argument("--torch-trace", type=str, default=None, help="with --torch-profile: also write a Chrome trace of rank 0")
    p.add_argument("--ep", type=int, default=1, help="expert-parallel size (mixture-of-experts models)")
    p.add_argument("--sample-max", type=int, default=4096, help="longest synthetic sample that is packed")
    p.add_argument("--no-cta-pairs", action="store_true", help="use the single-CTA 128x256 GEMM tile instead of the CTA-pair kernel")
    return p.parse_args()


def reference_unavailable() -> None:
    print(json.dumps({
        "impl": "reference",
        "unavailable": "reference cannot be installed offline: its build backend (hatchling) and its hard dependency "
                       "deepspeed are absent from the wheelhouse, and `import arctic_training` fails without deepspeed",
    }))


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.proc = None
        self.path = Path(tempfile.mkstemp(prefix="atb_clocks_", suffix=".csv")[1])

    def start(self) -> None:
        try:
            self.fh = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=self.fh, stderr=subprocess.DEVNULL,
            )
        except Exception:
            self.proc = None

    def stop(self, gpu_indices) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.fh.close()
        clocks, maxes, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.path.read_text().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                idx, sm, mx, power = int(parts[0]), float(parts[1]), float(parts[2]), float(parts[3])
            except ValueError:
                continue
            if idx not in gpu_indices or power < 300.0:  # only samples taken under load
                continue
            clocks.append(sm)
            maxes.append(mx)
            for n, v in zip(names, parts[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        try:
            self.path.unlink()
        except OSError:
            pass
        return {
            "sm_mhz": statistics.median(clocks) if clocks else None,
            "sm_max_mhz": max(maxes) if maxes else None,
            "reasons": sorted(reasons),
            "samples": len(clocks),
        }


def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        reference_unavailable()
        return

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("for --gpus N > 1 launch with torch.distributed.run (one process per GPU)")
    os.environ.setdefault("AT_LOG_LEVEL", "WARNING")
    os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")

    from arctictraining_b200 import ops
    from arctictraining_b200.comm.dist import init_distributed
    from arctictraining_b200.config.trainer import get_config
    from arctictraining_b200.ops import functional as F_ops
    from arctictraining_b200.registry import get_registered_trainer
    from arctictraining_b200.trainer.utils import to_device

    init_distributed(local_rank)
    F_ops.set_gemm_backend(args.gemm)
    from arctictraining_b200.ops import _ext

    _ext.require()
    torch.ops.atb200.set_gemm_cta_pairs(not args.no_cta_pairs)
    device = torch.device("cuda", torch.cuda.current_device())

    total_steps = args.warmup + args.steps
    rows_needed = (2 * total_steps + 4) * world
    workdir = Path(tempfile.gettempdir()) / f"atb200_bench_{os.getuid()}"
    hf_kwargs = {"num_hidden_layers": args.layers} if args.layers else {}
    recipe = {
        "type": "sft",
        "micro_batch_size": 1,
        "epochs": 1,
        "seed": 42,
        "expert_parallel_size": args.ep,
        "arctic_moe": "auto",
        "model": {"name_or_path": args.model, "dtype": "bf16", "attn_implementation": args.attn, "hf_config_kwargs": hf_kwargs},
        "data": {
            "sources": [{"type": "synthetic", "num_samples": rows_needed * 4, "min_length": 256, "max_length": min(args.sample_max, args.seq_len),
                         "prompt_fraction": 0.5, "seed": 1234}],
            "cache_dir": str(workdir / "cache"),
            "max_length": args.seq_len,
            "pack_samples": True,
            "pad_to": "max_length",
            "dl_num_workers": 0,
            "num_proc": 1,
        },
        "optimizer": {"lr": 1e-5, "weight_decay": 0.1},
        "scheduler": {"name": "constant"},
        "deepspeed": {"zero_optimization": {"stage": args.zero_stage}, "gradient_clipping": 1.0,
                      "activation_checkpoint_keep": args.keep},
        "train_log_iter_interval": 0,
        "train_log_metrics_path": str(workdir / f"metrics_{rank}.jsonl"),
        "logger": {"level": "WARNING"},
    }
    config = get_config(recipe)
    library = args.impl == "library_stack"
    trainer = get_registered_trainer(config.type)(config, mode="process-data" if library else "train")

    batches = []
    it = iter(trainer.train_dataloader)
    for _ in range(2 * total_steps):
        b = next(it)
        b.pop("packed_sample_seqlens", None)
        batches.append(b)
    tokens_per_step = batches[0]["input_ids"].numel() * world
    h2d_bytes = sum(v.numel() * v.element_size() for v in batches[0].values() if torch.is_tensor(v))
    if library:
        sys.path.insert(0, str(ROOT / "benchmarks"))
        import library_stack

        library_stack.run(args, batches, tokens_per_step, h2d_bytes, ClockSampler)
        return
    engine = trainer.model
    engine.train()

    def barrier():
        if world > 1:
            dist.barrier(device_ids=[device.index])
        torch.cuda.synchronize()

    def device_step(b):
        out = engine(**b, use_cache=False)
        engine.backward(out.loss)
        engine.step()
        return out.loss

    # ------------------------------------------------------------------ device-timed region
    dev_batches = [to_device(b, device) for b in batches[:total_steps]]
    for b in dev_batches[: args.warmup]:
        device_step(b)
    barrier()
    sampler = ClockSampler()
    if rank == 0:
        sampler.start()
    launches0 = ops.LAUNCH_COUNTER["native"]
    comm0 = dict(ops.COMM_COUNTER)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    prof = None
    if args.torch_profile and rank == 0:
        from torch.profiler import ProfilerActivity
        from torch.profiler import profile

        prof = profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA])
        prof.__enter__()
    start.record()
    for b in dev_batches[args.warmup :]:
        loss = device_step(b)
    end.record()
    if prof is not None:
        torch.cuda.synchronize()
        prof.__exit__(None, None, None)
        Path(args.torch_profile).write_text(prof.key_averages().table(sort_by="cuda_time_total", row_limit=60, max_name_column_width=90))
        if args.torch_trace:
            prof.export_chrome_trace(args.torch_trace)
    barrier()
    ms = start.elapsed_time(end)
    launches = ops.LAUNCH_COUNTER["native"] - launches0
    comm_launches = {k: int(v - comm0.get(k, 0)) for k, v in ops.COMM_COUNTER.items() if v - comm0.get(k, 0)}
    clocks = sampler.stop(set(range(world))) if rank == 0 else {}
    final_loss = float(loss)
    err = int(torch.ops.atb200.read_and_clear_error_flag(dev_batches[0]["input_ids"]))
    del dev_batches

    # ------------------------------------------------------------------ end-to-end through the trainer API
    e2e_ms = None
    if not args.skip_e2e:
        e2e_batches = batches[total_steps : 2 * total_steps]
        for b in e2e_batches[: args.warmup]:  # the same warm-up as the device-timed loop
            trainer.metrics.values.clear() if trainer.metrics.enabled else None
            trainer.step(dict(b))
        barrier()
        t0 = time.perf_counter()
        for b in e2e_batches[args.warmup : args.warmup + args.steps]:
            if trainer.metrics.enabled:
                trainer.metrics.values.clear()
            trainer.step(dict(b))  # H2D of the pinned batch, fwd, bwd, optimizer step, loss.item()
        barrier()
        e2e_ms = (time.perf_counter() - t0) * 1e3

    stats = torch.tensor([ms, e2e_ms if e2e_ms is not None else 0.0], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    ms, e2e_ms_max = float(stats[0]), float(stats[1])

    if rank == 0:
        ms_per_step = ms / args.steps
        value = tokens_per_step / (ms_per_step / 1e3)
        cfg = trainer.model_unwrapped.config
        result = {
            "metric": METRIC if args.model == "llama-3.1-8b" else args.model.replace("-", "_").replace(".", "_") + "_sft_tokens_per_s",
            "value": round(value, 1),
            "unit": "tokens/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": round(ms_per_step, 3),
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "bf16",
            "data": "synthetic uniform token ids, packed variable-length samples; random-init weights",
            "impl": "native",
            "config": {
                "model": args.model,
                "layers": cfg["num_hidden_layers"],
                "global_batch": world,
                "seq_len": args.seq_len,
                "parallelism": f"zero{args.zero_stage}-dp{world}" + (f"-ep{args.ep}" if args.ep > 1 else ""),
                "optimizer": "adamw fp32 master",
                "activation_checkpointing": True,
                "layers_keeping_activations": (engine._keep_state.get("kept_layers", 0) if args.keep == "auto"
                                               else min(int(args.keep), cfg["num_hidden_layers"])),
                "attention": args.attn,
                "attention_backward": ("own tcgen05 kernel" if args.attn == "native" and os.getenv("ATB200_ATTN_BWD", "native") == "native"
                                       else os.getenv("ATB200_ATTN_BWD", "library")),
                "fused_comm": bool(getattr(engine, "symm", None) is not None),
                "gemm": args.gemm + ("" if args.gemm != "tcgen05" else ("-1cta" if args.no_cta_pairs else "-2cta")),
                "l2_policy": "inputs larger than L2 (16 GB of weights streamed every step)",
                "valid": not args.layers,
            },
            "clocks": clocks,
            "gpu_launches": int(launches),
            "comm_kernel_launches": comm_launches,
            "final_loss": round(final_loss, 4),
            "kernel_error_flag": err,
            "keep_state": {k: (round(v / 2**30, 2) if isinstance(v, (int, float)) and v > 1e6 else v)
                           for k, v in engine._keep_state.items()},
            "max_memory_gb": round(torch.cuda.max_memory_allocated() / 2**30, 2),
        }
        if e2e_ms is not None:
            e2e_per_step = e2e_ms_max / args.steps
            result["e2e"] = {
                "value": round(tokens_per_step / (e2e_per_step / 1e3), 1),
                "unit": "tokens/s",
                "ms_per_step": round(e2e_per_step, 3),
                "h2d_bytes_per_step": int(h2d_bytes),
                "d2h_bytes_per_step": 4,
            }
        print(json.dumps(result), flush=True)
    if world > 1:
        dist.barrier(device_ids=[device.index])
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
