#!/usr/bin/env python
"""Times the bandwidth-bound kernels against their ATen counterparts and against the
measured HBM copy bandwidth.

    python benchmarks/elementwise_bench.py [--shape 13b] [--iters 10] [--peak-gbs 6544]

Shapes: (tokens, hidden, ffn) of the benchmark models at their micro-batch size.  Every
tensor is far larger than L2 (126 MB).  Reported per op: milliseconds (CUDA events, 3
warm-up calls), algorithmic bytes moved, achieved GB/s and its fraction of ``--peak-gbs``
(default: the pool's measured copy bandwidth).  Rows:

  rmsnorm fwd / bwd     two-pass kernels (default) and the row-resident ones
                        (``FLEXTRAIN_RMSNORM=rows``), ATen composition for reference
  layernorm fwd / bwd   row-resident kernels vs ``torch.nn.functional.layer_norm``
  swiglu fwd / bwd      separate kernels; the GEMM-epilogue form is timed as a GEMM
                        (``benchmarks/gemm_bench.py`` shapes) and not here
  bias + gelu fwd / bwd native vs ATen
  rope                  in place on the q and k heads of a packed QKV tensor
"""
import argparse
import os
import sys

import torch
import torch.nn.functional as TF

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flextrain_b200.ops import cuda_ops  # noqa: E402

SHAPES = {"7b": (16384, 4096, 11008), "13b": (32768, 5120, 13824), "70b": (8192, 8192, 28672),
          "small": (4096, 4096, 11008)}


def timed(fn, iters):
    for _ in range(3):
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
    ap.add_argument("--shape", default="13b", choices=sorted(SHAPES))
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--peak-gbs", type=float, default=6544.0)
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    T, H, F = SHAPES[args.shape]
    bf = torch.bfloat16
    torch.manual_seed(0)
    x = torch.randn(T, H, device=dev, dtype=bf, requires_grad=True)
    w = torch.ones(H, device=dev, dtype=bf, requires_grad=True)
    b = torch.zeros(H, device=dev, dtype=bf, requires_grad=True)
    dy = torch.randn(T, H, device=dev, dtype=bf)
    gu = torch.randn(T, 2 * F, device=dev, dtype=bf, requires_grad=True)
    dact = torch.randn(T, F, device=dev, dtype=bf)
    pre = torch.randn(T, F, device=dev, dtype=bf, requires_grad=True)
    bias_f = torch.zeros(F, device=dev, dtype=bf, requires_grad=True)
    unit = T * H * 2                        # bytes of one [tokens, hidden] bf16 tensor
    unit_f = T * F * 2

    def report(name, ms, nbytes):
        gbs = nbytes / ms / 1e6
        print(f"{name:34s} {ms:8.3f} ms  {nbytes / 1e9:7.2f} GB  {gbs:7.0f} GB/s  {gbs / args.peak_gbs:5.2f} of peak",
              flush=True)

    def fwd_bwd(name, make, grads, dout, fwd_bytes, bwd_bytes):
        with torch.no_grad():
            report(name + " fwd", timed(make, args.iters), fwd_bytes)
        out = make()
        report(name + " bwd", timed(lambda: torch.autograd.grad(out, grads, dout, retain_graph=True), args.iters),
               bwd_bytes)

    print(f"shape {args.shape}: tokens {T}, hidden {H}, ffn {F}; peak {args.peak_gbs:.0f} GB/s")
    fwd_bwd("rmsnorm two-pass", lambda: cuda_ops.rmsnorm(x, w, 1e-5), (x, w), dy, 2 * unit, 3 * unit)
    fwd_bwd("rmsnorm rows", lambda: cuda_ops.rmsnorm_rows(x, w, 1e-5), (x, w), dy, 2 * unit, 3 * unit)

    def aten_rms():
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * w.float()).to(bf)
    fwd_bwd("rmsnorm ATen composition", aten_rms, (x, w), dy, 2 * unit, 3 * unit)
    fwd_bwd("layernorm rows", lambda: cuda_ops.layernorm(x, w, b, 1e-5), (x, w, b), dy, 2 * unit, 3 * unit)
    fwd_bwd("layernorm ATen", lambda: TF.layer_norm(x, (H,), w, b, 1e-5), (x, w, b), dy, 2 * unit, 3 * unit)
    fwd_bwd("swiglu", lambda: cuda_ops.swiglu(gu), (gu,), dact, 3 * unit_f, 5 * unit_f)
    fwd_bwd("bias+gelu native", lambda: cuda_ops.bias_gelu(pre, bias_f), (pre, bias_f), dact, 2 * unit_f,
            3 * unit_f)
    fwd_bwd("bias+gelu ATen", lambda: TF.gelu(pre + bias_f, approximate="tanh"), (pre, bias_f), dact,
            2 * unit_f, 3 * unit_f)
    # rotary embedding in place on the q and k heads of a packed QKV row (MHA layout: 3 * hidden wide)
    from flextrain_b200.ops import reference as ref
    d, seq = 128, 4096
    heads = 2 * (H // d)
    qkv = torch.randn(T // seq, seq, 3 * H, device=dev, dtype=bf)
    cos, sin = ref.rope_tables(seq, d, 10000.0, device=dev)
    with torch.no_grad():
        report("rope in place (q and k heads)", timed(lambda: cuda_ops.rope_heads_inplace(qkv, cos, sin, heads, d),
                                                      args.iters), 2 * 2 * unit)
    from flextrain_b200.ops.native import cuda_lib
    print("error word", cuda_lib().ft_gemm_error())


if __name__ == "__main__":
    main()
