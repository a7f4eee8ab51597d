# SPDX-License-Identifier: Apache-2.0
"""ZeRO-3 parameter all-gather inside the first consuming GEMM: one tcgen05 launch in which a few staging CTAs copy the
q|k|v weight from the ranks that own its pieces (contiguous shards of the layer's flat parameter buffer, peer memory)
into this rank's full buffer, tile of 256 weight rows by tile, while the CTA pairs multiply the tiles that have
arrived — against gather-then-GEMM with the peer-memory pull kernel and with the NCCL all-gather.  CUDA-event timing,
L2 flushed between iterations, max over ranks.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29562 \
        benchmarks/zero3_gather_gemm_bench.py --tokens 8192

Reference behaviour replaced: prefetched parameter all-gathers of the external engine (bucket sizes in
arctic_training/config/trainer.py:421-430) followed by a library GEMM.
"""

import argparse
import json
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--out-features", type=int, default=6144, help="rows of the weight (q|k|v of Llama-3.1-8B)")
    ap.add_argument("--unit-elems", type=int, default=218112000, help="elements of the whole layer unit (Llama-3.1-8B layer)")
    ap.add_argument("--stage-ctas", type=int, default=8)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--out", default=None)
    args = ap.parse_args()

    import torch
    import torch.distributed as dist

    from arctictraining_b200.comm.dist import init_distributed
    from arctictraining_b200.comm.symm import SymmetricContext
    from arctictraining_b200.ops import _ext
    from arctictraining_b200.ops import functional as Fn

    init_distributed(int(os.environ.get("LOCAL_RANK", "0")))
    _ext.require()
    ops = torch.ops.atb200
    rank, P = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    M, K, N = args.tokens, args.hidden, args.out_features
    gran = 256 * P
    numel = (args.unit_elems + gran - 1) // gran * gran
    shard = numel // P
    w_off = 4096 * 8  # the weight does not start at the beginning of the unit
    symm = SymmetricContext(None)
    slab = symm.alloc("shards", shard, torch.bfloat16)
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    slab.tensor.copy_((torch.randn(shard, device=dev, generator=g) * 0.02).bfloat16())
    x = (torch.randn(M, K, device=dev, generator=g)).bfloat16()
    full_pull = torch.zeros(numel, device=dev, dtype=torch.bfloat16)
    full_fused = torch.zeros(numel, device=dev, dtype=torch.bfloat16)
    full_nccl = torch.zeros(numel, device=dev, dtype=torch.bfloat16)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    torch.cuda.synchronize()
    dist.barrier(device_ids=[dev.index])

    def weight(buf):
        return buf[w_off : w_off + N * K].view(N, K)

    def fused():
        return ops.gemm_bf16_gather_b(x, slab.ptrs, 0, shard, full_fused, w_off, N, args.stage_ctas)

    def pull_then_gemm():
        symm.all_gather(slab, 0, shard, full_pull)
        return Fn.gemm(x, weight(full_pull))

    def nccl_then_gemm():
        dist.all_gather_into_tensor(full_nccl, slab.tensor)
        return Fn.gemm(x, weight(full_nccl))

    def gemm_only():
        return Fn.gemm(x, weight(full_pull))

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

    ref = pull_then_gemm()
    got = fused()
    torch.cuda.synchronize()
    same_w = bool(torch.equal(weight(full_fused), weight(full_pull)))
    same_out = bool(torch.equal(got, ref))
    res = {"tokens": M, "ranks": P, "weight": [N, K], "unit_mb": round(numel * 2 / 2**20, 1), "stage_ctas": args.stage_ctas,
           "weight_bit_identical": same_w, "output_bit_identical": same_out,
           "fused_ms": timeit(fused), "pull_unit_then_gemm_ms": timeit(pull_then_gemm),
           "nccl_unit_then_gemm_ms": timeit(nccl_then_gemm), "gemm_only_ms": timeit(gemm_only)}
    assert int(ops.read_and_clear_error_flag(x)) == 0
    symm.check()
    flops = 2.0 * M * N * K
    link_bytes = (P - 1) / P * N * K * 2
    peak = 1653.4e12  # measured bf16 GEMM peak of this pod (burst), FLOP/s
    link = 770e9      # measured peer copy bandwidth, bytes/s per direction
    roof_ms = max(flops / peak, link_bytes / link) * 1e3
    res["roofline_ms"] = roof_ms
    res["fraction_of_roofline"] = roof_ms / res["fused_ms"]
    res["gemm_tflops_fused"] = flops / res["fused_ms"] / 1e9
    if rank == 0:
        print(json.dumps(res))
        if args.out:
            with open(args.out, "a") as f:
                f.write(json.dumps(res) + "\n")
    dist.barrier(device_ids=[dev.index])
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
