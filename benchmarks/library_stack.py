# SPDX-License-Identifier: Apache-2.0
"""Library-stack proxy for the headline benchmark (NOT the reference and none of this package's kernels or engine).

What a user gets on this machine from stock libraries for the same job: Hugging Face ``LlamaForCausalLM`` built from a
config (random weights) with flash-attn 2 attention (what the reference's recipes select), Liger fused linear
cross-entropy / RMSNorm / RoPE / SwiGLU, torch FSDP2 ``fully_shard`` (fp32 sharded parameters, bf16 compute, fp32
gradient reduction = ZeRO-3 with fp32 master weights), ``torch.optim.AdamW(fused=True)``, gradient clipping 1.0 and
Hugging Face gradient checkpointing (the reference's default).  The synthetic packed batches are the ones
``bench.py`` feeds to the native arm (same recipe, same seed), timed the same way (CUDA events, max over ranks).
The reference itself (DeepSpeed ZeRO-3 under the same Hugging Face model) cannot be installed here; this arm is its
stand-in for context and never labels itself "reference".

Called by ``bench.py --impl library_stack``.
"""

from __future__ import annotations

import json
import os
import time


def run(args, batches, tokens_per_step, h2d_bytes, sampler_cls) -> None:
    import torch
    import torch.distributed as dist
    from torch.distributed.fsdp import MixedPrecisionPolicy
    from torch.distributed.fsdp import fully_shard
    from transformers import LlamaConfig
    from transformers import LlamaForCausalLM

    from arctictraining_b200.models.arch import load_arch_config

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    device = torch.device("cuda", torch.cuda.current_device())
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29577")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)

    arch = load_arch_config(args.model, {"num_hidden_layers": args.layers} if args.layers else {})
    liger = False
    if not args.no_liger:
        try:
            from liger_kernel.transformers import apply_liger_kernel_to_llama

            apply_liger_kernel_to_llama(rope=True, cross_entropy=False, fused_linear_cross_entropy=True, rms_norm=True, swiglu=True)
            liger = True
        except Exception as exc:  # noqa: BLE001
            print(f"[library_stack] Liger patch unavailable: {exc}", flush=True)
    cfg = LlamaConfig(
        vocab_size=arch["vocab_size"], hidden_size=arch["hidden_size"], intermediate_size=arch["intermediate_size"],
        num_hidden_layers=arch["num_hidden_layers"], num_attention_heads=arch["num_attention_heads"],
        num_key_value_heads=arch["num_key_value_heads"], max_position_embeddings=arch["max_position_embeddings"],
        rms_norm_eps=arch["rms_norm_eps"], rope_parameters={"rope_type": "default", "rope_theta": arch["rope_theta"]},
        tie_word_embeddings=False, attn_implementation=args.library_attn, use_cache=False,
    )
    torch.manual_seed(42)
    with torch.device(device):
        model = LlamaForCausalLM(cfg).to(torch.float32)
    if not args.no_grad_ckpt:
        model.gradient_checkpointing_enable(gradient_checkpointing_kwargs={"use_reentrant": False})
    model.train()
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
    for layer in model.model.layers:
        fully_shard(layer, mp_policy=mp)
    fully_shard(model, mp_policy=mp)
    decay = [p for n, p in model.named_parameters() if p.ndim >= 2]
    no_decay = [p for n, p in model.named_parameters() if p.ndim < 2]
    opt = torch.optim.AdamW([{"params": decay, "weight_decay": 0.1}, {"params": no_decay, "weight_decay": 0.0}],
                            lr=1e-5, betas=(0.9, 0.999), fused=True)

    def step(b):
        out = model(input_ids=b["input_ids"], position_ids=b["position_ids"], labels=b["labels"], use_cache=False)
        out.loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        opt.zero_grad(set_to_none=True)
        return out.loss

    def barrier():
        if world > 1:
            dist.barrier(device_ids=[device.index])
        torch.cuda.synchronize()

    total = args.warmup + args.steps
    keys = ("input_ids", "position_ids", "labels")
    dev = [{k: b[k].to(device) for k in keys} for b in batches[:total]]
    for b in dev[: args.warmup]:
        step(b)
    barrier()
    sampler = sampler_cls()
    if rank == 0:
        sampler.start()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for b in dev[args.warmup :]:
        loss = step(b)
    end.record()
    barrier()
    ms = start.elapsed_time(end)
    clocks = sampler.stop(set(range(world))) if rank == 0 else {}
    final_loss = float(loss)
    del dev

    # end to end: pinned host batch -> device every step, loss read back every step
    e2e = batches[total : 2 * total]
    pinned = [{k: b[k].pin_memory() for k in keys} for b in e2e]
    for b in pinned[: args.warmup]:
        float(step({k: v.to(device, non_blocking=True) for k, v in b.items()}))
    barrier()
    t0 = time.perf_counter()
    for b in pinned[args.warmup : args.warmup + args.steps]:
        float(step({k: v.to(device, non_blocking=True) for k, v in b.items()}))
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3

    stats = torch.tensor([ms, e2e_ms], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    ms, e2e_ms = float(stats[0]), float(stats[1])
    if rank == 0:
        per = ms / args.steps
        e2e_per = e2e_ms / args.steps
        print(json.dumps({
            "metric": "llama3.1_8b_sft_tokens_per_s" if args.model == "llama-3.1-8b" else args.model + "_sft_tokens_per_s",
            "value": round(tokens_per_step / (per / 1e3), 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(per, 3), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic uniform token ids, packed variable-length samples; random-init weights",
            "impl": "library_stack",
            "note": "library-stack proxy, not the reference: transformers LlamaForCausalLM + flash-attn + Liger + FSDP2 + fused AdamW",
            "config": {
                "model": args.model, "layers": arch["num_hidden_layers"], "global_batch": world, "seq_len": args.seq_len,
                "parallelism": f"fsdp2-dp{world}", "optimizer": "torch AdamW fused, fp32 sharded parameters",
                "activation_checkpointing": not args.no_grad_ckpt, "attention": args.library_attn, "liger": liger,
                "l2_policy": "inputs larger than L2 (weights streamed every step)", "valid": not args.layers,
            },
            "clocks": clocks, "gpu_launches": 0, "final_loss": round(final_loss, 4),
            "max_memory_gb": round(torch.cuda.max_memory_allocated() / 2**30, 2),
            "e2e": {"value": round(tokens_per_step / (e2e_per / 1e3), 1), "unit": "tokens/s", "ms_per_step": round(e2e_per, 3),
                    "h2d_bytes_per_step": int(h2d_bytes), "d2h_bytes_per_step": 4},
        }), flush=True)
    if world > 1:
        dist.barrier(device_ids=[device.index])
    dist.destroy_process_group()
