#!/usr/bin/env python
"""The two fused compute + collective kernels on ONE GPU with emulated ranks, for profiler
captures and for a quick look at their device time without a multi-GPU box.

    python benchmarks/fused_emulated.py --what rs   [--world 8] [--numel 16M] [--iters 3]
    python benchmarks/fused_emulated.py --what ag   [--world 4] [--m 2048 --n 4096 --k 2048]
    python benchmarks/fused_emulated.py --what gather [--world 8] [--mib 256]

All "peer" buffers live on this GPU and every flag word already holds the call's sequence
number, so both barriers pass at once and one rank's kernel runs alone (kernels that wait on
one another must never run as separate launches on one device).  What the counters of such a
capture show is the kernel's own work - loads of `world` buffers, the fp32 sum, Adam, the
tensor-core tiles beside the copy warps - with HBM standing in for NVLink.
"""
import argparse
import ctypes
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flextrain_b200.ops.native import cuda_lib  # noqa: E402
from flextrain_b200.parallel import fused  # noqa: E402
from flextrain_b200.param_group import GroupSegment  # noqa: E402

SIZES = {"1M": 1 << 20, "16M": 1 << 24, "64M": 1 << 26, "256M": 1 << 28}


class Owner:
    defaults = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, bias_correction=True)
    adamw_mode = True


def timed(fn, iters):
    fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters


def flags(world, seq, dev):
    fl = [torch.full((128 * 8,), seq, dtype=torch.int32, device=dev) for _ in range(world)]
    return fl, (ctypes.c_void_p * world)(*[f.data_ptr() for f in fl])


def run_rs(args, dev):
    world, n = args.world, SIZES[args.numel] // (args.world * 8) * (args.world * 8)
    S = n // world
    grads = [torch.randn(n, device=dev).to(torch.bfloat16) for _ in range(world)]
    gp = (ctypes.c_void_p * world)(*[g.data_ptr() for g in grads])
    _keep, fp = flags(world, 1, dev)
    master, m, v = torch.randn(S, device=dev), torch.zeros(S, device=dev), torch.zeros(S, device=dev)
    out = torch.empty(S, device=dev, dtype=torch.bfloat16)
    segs = fused.make_segments([GroupSegment(0, 0, S)], [{}], Owner, 1)

    def call():
        fused.rs_adam(world, 0, gp, fp, torch.bfloat16, S, 1.0 / (world * 65536.0), 1, None, S, True, master,
                      m, v, out, S, None, torch.bfloat16, None, None, segs, 1, max_blocks=args.blocks)

    ms = timed(call, args.iters)
    assert fused.comm_error() == 0
    algo = S * (2 * world + 12 + 12 + 2)
    print(f"rs_adam emulated: world {world}, {n} gradient elements per rank, shard {S}: {ms:.4f} ms, "
          f"{algo / ms / 1e6:.0f} GB/s of algorithmic traffic ({algo / 1e6:.1f} MB: {world} bf16 slices read, "
          f"fp32 p/m/v read and written, bf16 parameter written)")


def run_ag(args, dev):
    world, M, N, K = args.world, args.m, args.n, args.k
    assert N % world == 0
    rows = N // world
    W = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16)
    x = torch.randn(M, K, device=dev).to(torch.bfloat16)
    bufs = []
    for r in range(world):
        b = torch.zeros(N, K, device=dev, dtype=torch.bfloat16)
        b[r * rows:(r + 1) * rows] = W[r * rows:(r + 1) * rows]
        bufs.append(b)
    wp = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])
    _keep, fp = flags(world, 1, dev)
    y = torch.empty(M, N, device=dev, dtype=torch.bfloat16)

    def call():
        fused.ag_gemm(world, 0, wp, fp, 1, x, N, out=y)

    ms = timed(call, args.iters)
    assert cuda_lib().ft_gemm_error() == 0
    err = ((y.float() - x.float() @ W.float().t()).norm() / (x.float() @ W.float().t()).norm()).item()
    flops = 2.0 * M * N * K
    print(f"ag_gemm emulated: world {world}, M {M} N {N} K {K}: {ms:.4f} ms, {flops / ms / 1e9:.0f} TF/s, "
          f"{(world - 1) * rows * K * 2 / 1e6:.1f} MB gathered, relative error {err:.2e}")


def run_gather(args, dev):
    world = args.world
    shard = (args.mib << 20) // world // 4096 * 4096
    bufs = [torch.randint(0, 255, (shard * world,), dtype=torch.uint8, device=dev) for _ in range(world)]
    bp = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])
    _keep, fp = flags(world, 1, dev)

    def call():
        fused.peer_gather(world, 0, bp, fp, 1, shard, num_copiers=args.blocks)

    ms = timed(call, args.iters)
    assert cuda_lib().ft_gemm_error() == 0
    moved = (world - 1) * shard
    print(f"peer_gather emulated: world {world}, {moved / 1e6:.1f} MB pulled: {ms:.4f} ms, "
          f"{2 * moved / ms / 1e6:.0f} GB/s read + written")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", required=True, choices=["rs", "ag", "gather"])
    ap.add_argument("--world", type=int, default=8)
    ap.add_argument("--numel", default="16M", choices=sorted(SIZES))
    ap.add_argument("--m", type=int, default=2048)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--mib", type=int, default=256)
    ap.add_argument("--blocks", type=int, default=148)
    ap.add_argument("--iters", type=int, default=3)
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    {"rs": run_rs, "ag": run_ag, "gather": run_gather}[args.what](args, dev)


if __name__ == "__main__":
    main()
