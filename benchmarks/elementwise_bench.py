# SPDX-License-Identifier: Apache-2.0
"""Bandwidth of the memory-bound kernels (RMSNorm, RoPE, SwiGLU, AdamW, squared norm, cross-entropy) on inputs larger
than L2, against the measured copy bandwidth.  CUDA events, median of `--iters`, a 256 MB L2 flush between iterations.

    python benchmarks/elementwise_bench.py --tokens 32768 [--only adamw] [--out file.jsonl]
"""

import argparse
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inter", type=int, default=14336)
    ap.add_argument("--vocab", type=int, default=32768, help="columns of the logits tile for the cross-entropy kernel")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--only", default=None)
    ap.add_argument("--out", default=None)
    args = ap.parse_args()

    from arctictraining_b200.ops import _ext

    _ext.require()
    k = torch.ops.atb200
    T, H, I, V = args.tokens, args.hidden, args.inter, args.vocab
    dev = "cuda"
    peaks = Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    hbm = json.loads(peaks.read_text())["hbm_gbs"] if peaks.exists() else 6650.0
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    x = torch.randn(T, H, device=dev).bfloat16()
    w = torch.ones(H, device=dev).bfloat16()
    dy = torch.randn(T, H, device=dev).bfloat16()
    y, rstd = k.rmsnorm_fwd(x, w, 1e-5)
    gu = torch.randn(T, 2 * I, device=dev).bfloat16()
    dh = torch.randn(T, I, device=dev).bfloat16()
    n = 256 * 1024 * 1024
    master, grad, m, v = (torch.randn(n, device=dev) * 0.01 for _ in range(4))
    v.abs_()
    lp = torch.empty(n, device=dev, dtype=torch.bfloat16)
    qkv = torch.randn(T, 6144, device=dev).bfloat16()
    pos = torch.arange(T, device=dev)[:, None].float() * (1.0 / 10000 ** (torch.arange(64, device=dev).float() / 64))[None]
    cos, sin = pos.cos().contiguous(), pos.sin().contiguous()
    logits = torch.randn(T // 4, V, device=dev).bfloat16()
    labels = torch.randint(0, V, (T // 4,), device=dev)

    cases = {
        # name: (callable, bytes read + written)
        "rmsnorm_fwd": (lambda: k.rmsnorm_fwd(x, w, 1e-5), 2 * T * H * 2),
        "rmsnorm_bwd": (lambda: k.rmsnorm_bwd(dy, x, w, rstd), 3 * T * H * 2),
        "rope_qkv": (lambda: k.rope_inplace(qkv.view(T, 48, 128)[:, :40], cos, sin, False), 2 * T * 5120 * 2),
        "swiglu_fwd": (lambda: k.swiglu_fwd(gu), 3 * T * I * 2),
        "swiglu_bwd": (lambda: k.swiglu_bwd(dh, gu), 5 * T * I * 2),
        "adamw": (lambda: k.adamw_step(master, grad, m, v, lp, 1e-4, 0.9, 0.95, 1e-8, 0.1, 1, None), n * (4 * 4 + 3 * 4 + 2)),
        "sumsq": (lambda: k.sumsq(grad), n * 4),
        "ce_fwd_bwd": (lambda: k.ce_fwd_bwd(logits, labels, None, None, True), 2 * logits.numel() * 2),
    }
    results = {}
    for name, (fn, nbytes) in cases.items():
        if args.only and args.only != name:
            continue
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
        ms = ts[len(ts) // 2]
        gbs = nbytes / ms / 1e6
        results[name] = {"ms": round(ms, 4), "GBps": round(gbs, 1), "of_measured_copy": round(gbs / hbm, 3)}
    print(json.dumps(results))
    if args.out:
        with open(args.out, "a") as f:
            f.write(json.dumps(results) + "\n")


if __name__ == "__main__":
    main()
