# SPDX-License-Identifier: Apache-2.0
"""Micro-benchmark of the tcgen05 GEMM against cuBLAS (torch.matmul) on the shapes of a Llama-3.1-8B layer.

    python benchmarks/gemm_bench.py                 # all shapes, forward / dgrad / wgrad layouts
    python benchmarks/gemm_bench.py --case 8192,4096,4096 --iters 3 --no-cublas   # small fixed case (profiling)

Timing: CUDA events on the launching stream after warm-up; operands of every case exceed the 126 MB L2.
"""

import argparse
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
from arctictraining_b200.ops import _ext  # noqa: E402

SHAPES = [(8192, 6144, 4096), (8192, 4096, 4096), (8192, 28672, 4096), (8192, 4096, 14336), (8192, 8192, 8192),
          (4096, 128256, 4096)]


def timeit(fn, iters, warm):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", type=str, default="")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--no-cublas", action="store_true")
    ap.add_argument("--out", type=str, default="")
    ap.add_argument("--pairs", action="store_true", help="use the CTA-pair (cta_group::2) kernel")
    args = ap.parse_args()
    _ext.require()
    k = torch.ops.atb200
    k.set_gemm_cta_pairs(bool(args.pairs))
    shapes = [tuple(int(x) for x in args.case.split(","))] if args.case else SHAPES
    rows = []
    for M, N, K in shapes:
        a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
        dy = torch.randn(M, N, device="cuda", dtype=torch.bfloat16)
        fl = 2 * M * N * K / 1e12
        r = {"M": M, "N": N, "K": K}
        r["fwd_tflops"] = round(fl / timeit(lambda: k.gemm_bf16(a, b, False, False, 0, None, 0), args.iters, args.warmup) * 1e3, 1)
        if not args.case:
            r["dgrad_tflops"] = round(fl / timeit(lambda: k.gemm_bf16(dy, b, False, True, 0, None, 0), args.iters, args.warmup) * 1e3, 1)
            r["wgrad_tflops"] = round(fl / timeit(lambda: k.gemm_bf16(dy, a, True, True, 0, None, 0), args.iters, args.warmup) * 1e3, 1)
        if not args.no_cublas:
            r["cublas_tflops"] = round(fl / timeit(lambda: torch.matmul(a, b.t()), args.iters, args.warmup) * 1e3, 1)
        print(json.dumps(r), flush=True)
        rows.append(r)
    print("kernel error flag:", int(k.read_and_clear_error_flag(a)))
    if args.out:
        Path(args.out).write_text(json.dumps(rows, indent=1))


if __name__ == "__main__":
    main()
