#!/usr/bin/env python
"""Timeline of one CTA of the attention backward (default) or forward kernel.

    python benchmarks/attn_timeline.py [--pass bwd|fwd] [--shape 13b] [--cta 0] [--it0 8]

Backward.  Runs the backward once with its timeline instantiation: the CTA ``--cta`` records
clock64() at every hand-over point of eight consecutive (head, query block)
iterations starting at ``--it0``.  Prints, per iteration, the clock of each point
relative to the moment the product warp begins that iteration, and the mean
iteration period.  The roles:

    load   0 dO buffer free | 1 Q buffer free
    mma    0 begin | 1 Q landed | 2 S columns free | 3 S, dP issued | 4 P written |
           5 dV issued | 6 dS written | 7 dK, dQ issued
    smx    0 begin | 1 S complete | 2 dS tile free again (after 6) | 3 S loaded | 4 P stored |
           5 P signalled | 6 dP complete | 7 dP loaded | 8 dS stored | 9 dS signalled |
           10 dQ complete | 11 dQ loaded, S released | 12 dQ staged, signalled
           (first / last softmax warp)
    red    0 dQ slabs full | 1 slabs inside the dS tile read | 2 all slabs read

Forward.  The CTA ``--cta`` (CTA 0 is the pair of query blocks with the most K/V blocks) records
eight consecutive K/V blocks j starting at ``--it0``:

    mma    0 begin of block j | 1 tile 0: V_j, P0_j and K_j+1 are there | 2 PV0(j) issued |
           3 QK0(j+1) issued | 4 tile 1: P1_j is there | 5 PV1(j) issued | 6 QK1(j+1) issued
    smx0 / smx1 (first softmax warp of tile 0 / 1)
           0 begin | 1 S complete | 2 S in registers | 3 row maximum known, O rescaled if needed |
           4 exponentials done, P stored | 5 P signalled
"""
import argparse
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flextrain_b200.ops.attention_backward import attention_backward  # noqa: E402
from flextrain_b200.ops.attention_native import attention_forward  # noqa: E402

SHAPES = {"one": (1, 4096, 1, 1, 128), "four": (1, 4096, 4, 4, 128), "small": (1, 4096, 16, 16, 128), "7b": (4, 4096, 32, 32, 128), "13b": (8, 4096, 40, 40, 128),
          "70b": (2, 4096, 64, 8, 128)}
ROLES = ("load", "mma", "smx-first", "smx-last", "red")
SITES = (2, 8, 13, 13, 3)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="13b")
    ap.add_argument("--cta", type=int, default=0)
    ap.add_argument("--it0", type=int, default=8)
    ap.add_argument("--pass", dest="which", default="bwd", choices=("bwd", "fwd"))
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    B, S, Hq, Hkv, D = SHAPES[args.shape]
    torch.manual_seed(0)
    mk = lambda h: torch.randn(B, S, h, D, device=dev, dtype=torch.bfloat16)  # noqa: E731
    q, k, v, do = mk(Hq), mk(Hkv), mk(Hkv), mk(Hq)
    scale = 1.0 / math.sqrt(D)
    if args.which == "fwd":
        for _ in range(2):
            attention_forward(q, k, v, scale)
        buf = torch.zeros(3 * 8 * 8, dtype=torch.int64, device=dev)
        attention_forward(q, k, v, scale, trace=(buf, args.cta, args.it0))
        torch.cuda.synchronize()
        t = buf.cpu().view(3, 8, 8)
        base = t[0, 0]
        print(f"forward, shape {args.shape} cta {args.cta} K/V blocks {args.it0}..{args.it0 + 7}")
        period = (base[1:] - base[:-1]).float()
        print("block period (clocks):", [int(x) for x in period], "mean", int(period.mean()))
        for r, (name, sites) in enumerate((("mma", 7), ("smx0", 6), ("smx1", 6))):
            for j in range(8):
                print(f"{name:9s} j+{j}: {[int(t[r, s_, j] - base[j]) for s_ in range(sites)]}")
        return
    o, lse, _ = attention_forward(q, k, v, scale)
    for _ in range(2):
        attention_backward(q, k, v, o, lse, do, scale)
    buf = torch.zeros(5 * 16 * 8, dtype=torch.int64, device=dev)
    attention_backward(q, k, v, o, lse, do, scale, trace=(buf, args.cta, args.it0))
    torch.cuda.synchronize()
    t = buf.cpu().view(5, 16, 8)
    base = t[1, 0]                                   # product warp begins the iteration
    print(f"shape {args.shape} cta {args.cta} iterations {args.it0}..{args.it0 + 7}")
    period = (base[1:] - base[:-1]).float()
    print("iteration period (clocks):", [int(x) for x in period], "mean", int(period.mean()))
    for r, name in enumerate(ROLES):
        for j in range(8):
            rel = [int(t[r, s_, j] - base[j]) for s_ in range(SITES[r])]
            print(f"{name:9s} it+{j}: {rel}")


if __name__ == "__main__":
    main()
