# SPDX-License-Identifier: Apache-2.0
"""Times the package's sm_100a flash-attention forward and backward kernels against library kernels (flash-attn 2;
cuDNN's fused backward for a single unpacked sequence) on packed causal GQA shapes (CUDA events, L2 flushed between
iterations).  Backward FLOPs are counted as 2.5 x the forward's.

    python benchmarks/attn_bench.py --seqlens 8192 --heads 32 --kv-heads 8 --iters 10 --backward
"""

import argparse
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--seqlens", type=str, default="8192", help="comma-separated packed sample lengths")
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-library", action="store_true")
    ap.add_argument("--backward", action="store_true", help="also time the backward kernels")
    ap.add_argument("--out", type=str, default=None)
    args = ap.parse_args()

    from arctictraining_b200.ops import _ext

    _ext.require()
    ops = torch.ops.atb200
    lens = [int(x) for x in args.seqlens.split(",")]
    T, Hq, Hkv, D = sum(lens), args.heads, args.kv_heads, 128
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device="cuda", dtype=torch.int32)
    qkv = torch.randn(T, (Hq + 2 * Hkv) * D, device="cuda", dtype=torch.bfloat16)
    q = qkv[:, : Hq * D].view(T, Hq, D)
    k = qkv[:, Hq * D : (Hq + Hkv) * D].view(T, Hkv, D)
    v = qkv[:, (Hq + Hkv) * D :].view(T, Hkv, D)
    scale = D ** -0.5
    flops = sum(4.0 * L * L * Hq * D / 2 for L in lens)  # causal: half of the square
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def timeit(fn):
        for _ in range(args.warmup):
            fn()
        ts = []
        for _ in range(args.iters):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        ts.sort()
        return ts[len(ts) // 2]

    res = {"seqlens": lens, "heads": Hq, "kv_heads": Hkv}
    ms = timeit(lambda: ops.fmha_fwd(q, k, v, cu, T // 128 + len(lens), scale))
    assert int(ops.read_and_clear_error_flag(q)) == 0
    res["native_ms"] = ms
    res["native_tflops"] = flops / ms / 1e9
    if not args.no_library:
        from flash_attn import flash_attn_varlen_func

        ms2 = timeit(lambda: flash_attn_varlen_func(q, k, v, cu, cu, max(lens), max(lens), causal=True, softmax_scale=scale))
        res["flash_attn_ms"] = ms2
        res["flash_attn_tflops"] = flops / ms2 / 1e9
    if args.backward:
        nblk = T // 128 + len(lens)
        out, lse = ops.fmha_fwd(q, k, v, cu, nblk, scale)
        g = torch.randn(T, Hq, D, device="cuda", dtype=torch.bfloat16)
        ms = timeit(lambda: ops.fmha_bwd(g, q, k, v, out, lse, cu, nblk, scale))
        assert int(ops.read_and_clear_error_flag(q)) == 0
        res["native_bwd_ms"] = ms
        res["native_bwd_tflops"] = 2.5 * flops / ms / 1e9
        if not args.no_library:
            from flash_attn.flash_attn_interface import _flash_attn_varlen_backward

            dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
            ms2 = timeit(lambda: _flash_attn_varlen_backward(
                g, q, k, v, out, lse, dq, dk, dv, cu, cu, max(lens), max(lens), 0.0, scale, True, -1, -1, 0.0, None, False))
            res["flash_attn_bwd_ms"] = ms2
            res["flash_attn_bwd_tflops"] = 2.5 * flops / ms2 / 1e9
            if len(lens) == 1:
                from arctictraining_b200.ops.functional import _cudnn_dense_attention_backward
                from arctictraining_b200.ops.functional import _cudnn_dense_backward_applicable

                if _cudnn_dense_backward_applicable(q, k, v):
                    ms3 = timeit(lambda: _cudnn_dense_attention_backward(g, q, k, v, out, lse, 1, scale))
                    res["cudnn_bwd_ms"] = ms3
                    res["cudnn_bwd_tflops"] = 2.5 * flops / ms3 / 1e9
    print(json.dumps(res))
    if args.out:
        with open(args.out, "a") as f:
            f.write(json.dumps(res) + "\n")


if __name__ == "__main__":
    main()
