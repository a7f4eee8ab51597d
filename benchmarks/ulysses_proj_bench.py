# SPDX-License-Identifier: Apache-2.0
"""Head -> sequence exchange + output projection: one tcgen05 GEMM launch in which a few CTAs gather the
A operand from the peers' memory over NVLink while the others multiply the row tiles that have arrived (and the variant
where every CTA pair fetches its A tiles from the owners with TMA) against the two-step version (exchange kernel, barrier,
copy, local GEMM) and against NCCL all-to-all + GEMM.  CUDA-event timing, max over ranks.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29561 \
        benchmarks/ulysses_proj_bench.py --tokens 131072
"""

import argparse
import json
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=131072, help="tokens of the whole sequence")
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--out", default=None)
    args = ap.parse_args()

    import torch
    import torch.distributed as dist

    from arctictraining_b200.comm.dist import init_distributed
    from arctictraining_b200.ops import _ext
    from arctictraining_b200.ops import functional as Fn
    from arctictraining_b200.parallel import ulysses as U

    init_distributed(int(os.environ.get("LOCAL_RANK", "0")))
    _ext.require()
    rank, P = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    S, D = args.tokens, 128
    S_loc, Hl = S // P, args.heads // P
    torch.manual_seed(rank)
    y = torch.randn(S, Hl, D, device=dev, dtype=torch.bfloat16)          # my heads, all tokens
    w = (torch.randn(args.hidden, args.heads * D, device=dev) * 0.02).bfloat16()
    ex = U._PeerExchange(dist.group.WORLD)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def fused():
        return ex.head_to_seq_project(y, w, None)[0]

    def fused_direct():
        return ex.head_to_seq_project(y, w, None, stage_ctas=0)[0]

    def two_step():
        return Fn.gemm(ex.head_to_seq(y).view(S_loc, args.heads * D), w)

    def nccl():
        return Fn.gemm(U._head_to_seq(y[None], dist.group.WORLD).reshape(S_loc, args.heads * D), w)

    def timeit(fn):
        for _ in range(args.warmup):
            fn()
        ts = []
        for _ in range(args.iters):
            flush.zero_()
            dist.barrier(device_ids=[dev.index])
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        ts.sort()
        t = torch.tensor([ts[len(ts) // 2]], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    ref = two_step().float()
    err = float((fused().float() - ref).norm() / ref.norm())
    res = {"tokens": S, "ranks": P, "rel_err_fused_vs_two_step": err,
           "fused_ms": timeit(fused), "fused_direct_tma_ms": timeit(fused_direct), "two_step_ms": timeit(two_step), "nccl_ms": timeit(nccl)}
    ex.symm.check()
    flops = 2.0 * S_loc * args.hidden * args.heads * D
    link_bytes = (P - 1) / P * S_loc * args.heads * D * 2
    res["gemm_tflops_fused"] = flops / res["fused_ms"] / 1e9
    res["link_gbs_fused"] = link_bytes / res["fused_ms"] / 1e6
    if rank == 0:
        print(json.dumps(res))
        if args.out:
            with open(args.out, "a") as f:
                f.write(json.dumps(res) + "\n")
    dist.barrier(device_ids=[dev.index])
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
