#!/usr/bin/env python
"""Times the native causal attention kernels against PyTorch SDPA.

    python benchmarks/attn_bench.py [--shapes 7b 13b 70b small] [--iters 5] [--no-sdpa]
                                    [--pass fwd bwd]

Shapes are (batch, seq, q heads, kv heads, head dim).  CUDA events, 3 warm-up
launches; q/k/v/o/do of the named shapes are larger than L2 except for
``small``, which exists for profiler captures.  FLOPs are the causal ones
(half of the dense count): forward 4*B*H*S^2*D/2, backward 2.5x that.
"""
import argparse
import math
import os
import sys

import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flextrain_b200.ops.attention_native import attention_native  # noqa: E402

SHAPES = {
    "small": (1, 4096, 16, 16, 128),
    "7b": (4, 4096, 32, 32, 128),
    "13b": (8, 4096, 40, 40, 128),
    "70b": (2, 4096, 64, 8, 128),
}


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
    ap.add_argument("--shapes", nargs="+", default=["7b", "13b", "70b"])
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--no-sdpa", action="store_true")
    ap.add_argument("--pass", dest="passes", nargs="+", default=["fwd", "bwd"])
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    from flextrain_b200.ops.native import cuda_lib
    for name in args.shapes:
        B, S, Hq, Hkv, D = SHAPES[name]
        torch.manual_seed(0)
        mk = lambda h: torch.randn(B, S, h, D, device=dev, dtype=torch.bfloat16, requires_grad=True)  # noqa: E731
        q, k, v = mk(Hq), mk(Hkv), mk(Hkv)
        do = torch.randn(B, S, Hq, D, device=dev, dtype=torch.bfloat16)
        scale = 1.0 / math.sqrt(D)
        fwd_flops = 4.0 * B * Hq * S * S * D / 2
        line = [f"{name} B={B} S={S} Hq={Hq} Hkv={Hkv} D={D}:"]
        if "fwd" in args.passes:
            with torch.no_grad():
                ms = timed(lambda: attention_native(q, k, v, scale), args.iters)
            line.append(f"fwd native {ms:.3f} ms {fwd_flops / ms / 1e9:.0f} TF/s")
            if not args.no_sdpa:
                qh, kh, vh = (x.permute(0, 2, 1, 3) for x in (q, k, v))
                with torch.no_grad():
                    ms = timed(lambda: F.scaled_dot_product_attention(
                        qh, kh, vh, is_causal=True, enable_gqa=Hq != Hkv), args.iters)
                line.append(f"sdpa {ms:.3f} ms {fwd_flops / ms / 1e9:.0f} TF/s |")
        if "bwd" in args.passes:
            o = attention_native(q, k, v, scale)
            ms = timed(lambda: torch.autograd.grad(o, (q, k, v), do, retain_graph=True), args.iters)
            line.append(f"bwd native {ms:.3f} ms {2.5 * fwd_flops / ms / 1e9:.0f} TF/s")
            if not args.no_sdpa:
                qh, kh, vh = (x.permute(0, 2, 1, 3) for x in (q, k, v))
                o2 = F.scaled_dot_product_attention(qh, kh, vh, is_causal=True, enable_gqa=Hq != Hkv)
                doh = do.permute(0, 2, 1, 3)
                ms = timed(lambda: torch.autograd.grad(o2, (q, k, v), doh, retain_graph=True), args.iters)
                line.append(f"sdpa {ms:.3f} ms {2.5 * fwd_flops / ms / 1e9:.0f} TF/s")
        print(" ".join(line), flush=True)
    print("error word", cuda_lib().ft_gemm_error())


if __name__ == "__main__":
    main()
