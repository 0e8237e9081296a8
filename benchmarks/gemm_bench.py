#!/usr/bin/env python
"""Times the tcgen05 GEMM against torch.matmul (cuBLAS) on the Llama shapes.

    python benchmarks/gemm_bench.py [--shapes 70b|13b|7b|8k|small] [--iters 10]

CUDA events, 3 warm-up launches, a >L2 buffer is rewritten between timed
launches.  Prints one line per (shape, layout): ms, TFLOP/s, fraction of the
cuBLAS time, and the fraction of the measured bf16 peak from
MEASURED_PEAKS.json when that file is present.
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flextrain_b200.ops.cuda_ops import gemm  # noqa: E402

SHAPES = {
    "small": [(4096, 4096, 4096)],
    "8k": [(8192, 8192, 8192)],
    "7b": [(16384, 12288, 4096), (16384, 4096, 4096), (16384, 22016, 4096), (16384, 4096, 11008)],
    "13b": [(32768, 15360, 5120), (32768, 5120, 5120), (32768, 27648, 5120), (32768, 5120, 13824)],
    "70b": [(8192, 10240, 8192), (8192, 8192, 8192), (8192, 57344, 8192), (8192, 8192, 28672),
            (16384, 28672, 8192)],
}


def timed(fn, iters, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        total += s.elapsed_time(e)
    return total / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="70b")
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args()
    peak = None
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        peak = json.load(open(path)).get("bf16_tflops")
    dev = torch.device("cuda", 0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for (m, n, k) in SHAPES[args.shapes]:
        x = torch.randn(m, k, device=dev, dtype=torch.bfloat16)
        w = torch.randn(n, k, device=dev, dtype=torch.bfloat16)
        dy = torch.randn(m, n, device=dev, dtype=torch.bfloat16)
        y = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
        dx = torch.empty(m, k, device=dev, dtype=torch.bfloat16)
        dw = torch.empty(n, k, device=dev, dtype=torch.bfloat16)
        cases = [
            ("fwd  y=x.wT", lambda: gemm(x, False, w, False, m, n, k, out=y), lambda: torch.matmul(x, w.t(), out=y)),
            ("dgrad dx=dy.w", lambda: gemm(dy, False, w, True, m, k, n, out=dx), lambda: torch.matmul(dy, w, out=dx)),
            ("wgrad dw=dyT.x", lambda: gemm(dy, True, x, True, n, k, m, out=dw), lambda: torch.matmul(dy.t(), x, out=dw)),
        ]
        flops = 2.0 * m * n * k
        for name, ours, lib in cases:
            t_ours = timed(ours, args.iters, flush)
            t_lib = timed(lib, args.iters, flush)
            line = (f"M={m} N={n} K={k} {name:15s} ours {t_ours:8.3f} ms {flops / t_ours / 1e9:7.1f} TF/s | "
                    f"cuBLAS {t_lib:8.3f} ms {flops / t_lib / 1e9:7.1f} TF/s | ours/cuBLAS time {t_ours / t_lib:5.2f}")
            if peak:
                line += f" | {flops / t_ours / 1e9 / peak:5.2f} of measured peak"
            print(line, flush=True)


if __name__ == "__main__":
    main()
