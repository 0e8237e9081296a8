#!/usr/bin/env python
"""Clocks per 128-deep tcgen05 product for the operand placements of the attention kernels.

    python benchmarks/mma_rate.py [--rounds 2000]

Runs ``ft_mma_probe`` (csrc/kernels/mma_probe.cu) in each mode: one CTA per SM issues
``--rounds`` products of eight 128xNx16 instructions back to back on fixed tiles and times
them with clock64(); modes 5 and 6 put between the products what a pipelined kernel has
there (a barrier wait, a fence, a commit).  Prints the median over the CTAs of clocks per product, and the fraction
of the tensor pipe's rate that is (a 128x128x128 product is 512 clocks at 8192 dense bf16
FLOP per clock and SM, a 128x256x128 product 1024).
"""
import argparse
import ctypes
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flextrain_b200.ops.native import cuda_lib, ptr, stream_handle  # noqa: E402

MODES = (
    (0, 128, "A, B K-major in shared memory (S = Q K^T, dP = dO V^T); nothing between the products"),
    (1, 128, "A, B MN-major in shared memory (dV = P^T dO, dK = dS^T Q)"),
    (2, 128, "A K-major, B MN-major in shared memory (dQ = dS K)"),
    (3, 128, "A in tensor memory, B MN-major (O += P V)"),
    (4, 256, "A, B K-major in shared memory, N = 256"),
    (5, 128, "mode 0 + per product: barrier wait, fence, commit; issued inside `if (lane == 0)`"),
    (6, 128, "mode 0 + per product: barrier wait, fence, commit; whole warp, elected issuer"),
    (7, 128, "mode 0 while four warps keep loading tensor memory"),
    (8, 128, "mode 0 while four warps keep storing to shared memory"),
    (9, 128, "mode 3 while four warps keep loading tensor memory"),
    (10, 128, "mode 6 with the next product's barrier looked at between this product's 6th and 7th instruction"),
    (11, 128, "mode 0 while eight warps keep computing exponentials"),
    (12, 128, "mode 3 while eight warps keep computing exponentials"),
    (13, 128, "mode 3 while four warps keep storing to the tensor-memory columns A is read from"),
    (14, 256, "pair per round: O += P V (P in columns 0-63), then S = Q K^T over columns 0-127 (clocks per pair)"),
    (15, 256, "the same pair with S written to other columns (clocks per pair)"),
)

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rounds", type=int, default=2000)
    args = ap.parse_args()
    lib = cuda_lib()
    lib.ft_mma_probe.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    lib.ft_mma_probe.restype = ctypes.c_int
    dev = torch.device("cuda", 0)
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    out = torch.zeros(sms + 1, dtype=torch.int64, device=dev)
    for mode, n, what in MODES:
        for _ in range(2):                               # the first run warms up
            out.zero_()
            rc = lib.ft_mma_probe(mode, args.rounds, ptr(out), stream_handle())
            if rc != 0:
                raise SystemExit(f"ft_mma_probe({mode}) returned {rc}")
            torch.cuda.synchronize()
        per = out[:sms].float() / args.rounds
        med = per.median().item()
        ideal = 512.0 * n / 128
        print(f"mode {mode}: {med:7.1f} clocks per product (min {per.min().item():.1f}, max {per.max().item():.1f}), "
              f"{ideal / med:5.2f} of the pipe's rate  - {what}", flush=True)
    print("error word", lib.ft_gemm_error())


if __name__ == "__main__":
    main()
