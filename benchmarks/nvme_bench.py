#!/usr/bin/env python
"""Read / write rate of the NVMe engine as a function of how much is moved.

    python benchmarks/nvme_bench.py [--dir /tmp/ft_b200_swap] [--sizes-mib 256 1024 4096] [--stream-gib 16]

For each size: one file of that size written and read back three times through the engine the
training run uses (io_uring with O_DIRECT where the kernel grants it), median rate.  Then a
stream: ``--stream-gib`` GiB written as consecutive 1 GiB files and read back in the same order,
which is what optimizer state on the NVMe tier looks like to the disk - the rate of the whole
stream is the one a plan should count on.  Host memory only; no GPU work.
"""
import argparse
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flextrain_b200.memory.nvme_swapper import NVMeEngine  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--dir", default="/tmp/ft_b200_swap")
    ap.add_argument("--sizes-mib", type=int, nargs="+", default=[256, 1024, 4096])
    ap.add_argument("--stream-gib", type=int, default=16)
    args = ap.parse_args()
    os.makedirs(args.dir, exist_ok=True)
    eng = NVMeEngine()
    print(f"engine: {eng.kind}", flush=True)
    gib = 1 << 30
    for mib in args.sizes_mib:
        n = mib << 20
        buf = torch.empty(n, dtype=torch.uint8).fill_(7)
        path = os.path.join(args.dir, f"bench_{mib}.swp")
        tw, tr = [], []
        for _ in range(3):
            t0 = time.perf_counter(); eng.write(path, buf); tw.append(time.perf_counter() - t0)
        for _ in range(3):
            t0 = time.perf_counter(); eng.read(path, buf); tr.append(time.perf_counter() - t0)
        eng.forget(path)
        os.remove(path)
        print(f"{mib:6d} MiB: write {n / sorted(tw)[1] / 1e9:6.2f} GB/s, read {n / sorted(tr)[1] / 1e9:6.2f} GB/s "
              f"(first write {n / tw[0] / 1e9:.2f}, first read {n / tr[0] / 1e9:.2f})", flush=True)
    buf = torch.empty(gib, dtype=torch.uint8).fill_(3)
    paths = [os.path.join(args.dir, f"stream_{i}.swp") for i in range(args.stream_gib)]
    t0 = time.perf_counter()
    for p in paths:
        eng.write(p, buf)
    tw = time.perf_counter() - t0
    t0 = time.perf_counter()
    for p in paths:
        eng.read(p, buf)
    tr = time.perf_counter() - t0
    for p in paths:
        eng.forget(p)
        os.remove(p)
    total = args.stream_gib * gib
    print(f"stream of {args.stream_gib} x 1 GiB: write {total / tw / 1e9:.2f} GB/s, read {total / tr / 1e9:.2f} GB/s")
    eng.close()


if __name__ == "__main__":
    main()
