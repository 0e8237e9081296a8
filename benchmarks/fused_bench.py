#!/usr/bin/env python
"""Microbenchmarks of the two fused compute + collective kernels against the
NCCL (+cuBLAS / PyTorch) path, device-timed, max over ranks.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 \
        benchmarks/fused_bench.py [--what rs ag] [--sizes 1M 16M 256M 1B]

(a) rs: every rank holds a flat bf16 gradient of N elements (N(0,1), loss scale
    65536) and fp32 master / Adam moments of its N/world shard.  Fused =
    ``ft_rs_adam`` (peer reduce-scatter + unscale + Adam in one kernel);
    baseline = NCCL ``reduce_scatter_tensor`` + unscale + ``torch.optim.Adam(fused=True)``.
    Roofline: bytes entering the rank over NVLink at 770 GB/s (measured peer-copy
    bandwidth of this pool) vs HBM traffic at the measured copy bandwidth.
(b) ag: W[28672, 8192] bf16 row-sharded over the ranks, x[16384, 8192].  Fused =
    ``ft_ag_gemm``; baseline = NCCL ``all_gather_into_tensor`` + ``torch.matmul``.
    Roofline: the slower of FLOPs at the measured bf16 peak and inbound bytes at
    770 GB/s.
CUDA events, 3 warm-ups, a buffer larger than L2 is rewritten between iterations.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as tdist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import flextrain_b200 as ft  # noqa: E402
from flextrain_b200.parallel import fused  # noqa: E402
from flextrain_b200.parallel.symm_mem import FlagPage, SymmetricBuffer  # noqa: E402
from flextrain_b200.param_group import GroupSegment  # noqa: E402

NVLINK_GBS = 770.0
SIZES = {"1M": 1 << 20, "16M": 1 << 24, "256M": 1 << 28, "1B": 1 << 30}


def peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return p.get("hbm_gbs", 6650.0), p.get("bf16_tflops", 1590.0), "measured"
    return 6650.0, 1590.0, "fallback"


def timed(fn, iters, flush, world):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush.zero_()
        tdist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        total += s.elapsed_time(e)
    t = torch.tensor([total / iters], device="cuda")
    tdist.all_reduce(t, tdist.ReduceOp.MAX)
    return t.item()


class Owner:
    defaults = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, bias_correction=True)
    adamw_mode = True


def bench_rs(world, rank, dev, page, n, iters, flush, blocks):
    hbm, _, src = peaks()
    n = n // (world * 8) * (world * 8)
    S = n // world
    symm = SymmetricBuffer(n * 2)
    g = symm.tensor(torch.bfloat16)
    torch.manual_seed(rank)
    g.copy_(torch.randn(n, device=dev).to(torch.bfloat16))
    master = torch.randn(S, device=dev)
    m, v = torch.zeros(S, device=dev), torch.zeros(S, device=dev)
    out = torch.empty(S, device=dev, dtype=torch.bfloat16)
    segs = fused.make_segments([GroupSegment(0, 0, S)], [{}], Owner, 1)
    scale = 1.0 / (world * 65536.0)

    def run_fused():
        fused.rs_adam(world, rank, symm.ptr_array(), page.ptr_array(), torch.bfloat16, S, scale,
                      page.next_seq("b"), None, S, True, master, m, v, out, S, None, torch.bfloat16, None,
                      None, segs, 1, max_blocks=blocks)

    p_ref = torch.nn.Parameter(master.clone())
    opt = torch.optim.Adam([p_ref], lr=1e-3, fused=True)
    shard = torch.empty(S, device=dev, dtype=torch.bfloat16)
    gl = g.clone()

    def run_nccl():
        tdist.reduce_scatter_tensor(shard, gl, tdist.ReduceOp.SUM)
        p_ref.grad = shard.float().mul_(scale)
        opt.step()
        out.copy_(p_ref.data)

    t_f = timed(run_fused, iters, flush, world)
    t_n = timed(run_nccl, iters, flush, world)
    link_bytes = (world - 1) * S * 2
    hbm_bytes = S * (2 + 12 + 12 + 2)
    roof_ms = max(link_bytes / (NVLINK_GBS * 1e9), hbm_bytes / (hbm * 1e9)) * 1e3
    assert fused.comm_error() == 0
    symm.close()
    return {"bench": "rs_unscale_adam", "n": n, "world": world, "fused_ms": t_f, "nccl_torch_ms": t_n,
            "roofline_ms": roof_ms, "fused_frac_of_roofline": roof_ms / t_f,
            "nccl_frac_of_roofline": roof_ms / t_n, "speedup_vs_nccl": t_n / t_f, "peaks": src,
            "blocks": blocks}


def bench_ag(world, rank, dev, page, iters, flush):
    _, tf, src = peaks()
    M, N, K = 16384, 28672, 8192
    symm = SymmetricBuffer(N * K * 2)
    w = symm.tensor(torch.bfloat16).view(N, K)
    rows = N // world
    torch.manual_seed(0)
    full = (torch.randn(N, K, device=dev) * 0.02).to(torch.bfloat16)
    x = torch.randn(M, K, device=dev).to(torch.bfloat16)
    y = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
    shard = full[rank * rows:(rank + 1) * rows].contiguous()

    def reset():
        w.zero_()
        w[rank * rows:(rank + 1) * rows].copy_(shard)

    def run_fused():
        fused.ag_gemm(world, rank, symm.ptr_array(), page.ptr_array(), page.next_seq("ag"), x, N, out=y)

    gathered = torch.empty(N, K, device=dev, dtype=torch.bfloat16)

    def run_nccl():
        tdist.all_gather_into_tensor(gathered, shard)
        torch.matmul(x, gathered.t(), out=y)

    reset()
    torch.cuda.synchronize()
    tdist.barrier()
    run_fused()
    torch.cuda.synchronize()
    want = x.float()[:256] @ full.float().t()
    err = ((y[:256].float() - want).norm() / want.norm()).item()
    t_f = timed(run_fused, iters, flush, world)
    t_n = timed(run_nccl, iters, flush, world)
    flops = 2.0 * M * N * K
    link_bytes = (world - 1) * rows * K * 2
    roof_ms = max(flops / (tf * 1e12), link_bytes / (NVLINK_GBS * 1e9)) * 1e3
    from flextrain_b200.ops.native import cuda_lib
    assert cuda_lib().ft_gemm_error() == 0
    symm.close()
    return {"bench": "ag_gemm", "M": M, "N": N, "K": K, "world": world, "fused_ms": t_f,
            "nccl_cublas_ms": t_n, "roofline_ms": roof_ms, "fused_frac_of_roofline": roof_ms / t_f,
            "nccl_frac_of_roofline": roof_ms / t_n, "speedup_vs_nccl": t_n / t_f, "rel_err": err,
            "peaks": src, "form": "CTA pairs, one copy warp per CTA"}


def bench_gather(world, rank, dev, page, nbytes, iters, flush, blocks):
    """Whole-unit gather as the engine issues it: every rank owns 1/world of a flat buffer of
    ``nbytes`` (the bf16 parameters of one layer) and pulls the rest from its peers.
    ``ft_peer_gather`` against NCCL ``all_gather_into_tensor``; the roofline is
    the inbound bytes at the measured peer-copy rate."""
    from flextrain_b200.ops.native import cuda_lib
    shard = nbytes // world // 4096 * 4096
    symm = SymmetricBuffer(shard * world)
    flat = symm.tensor(torch.uint8)
    flat.random_(0, 255)
    mine = flat[rank * shard:(rank + 1) * shard].clone()
    gathered = torch.empty(shard * world, dtype=torch.uint8, device=dev)
    lib = cuda_lib()
    res = {"bench": "unit_gather", "bytes": shard * world, "world": world, "blocks": blocks}

    def run_peer():
        fused.peer_gather(world, rank, symm.ptr_array(), page.ptr_array(), page.next_seq("pg"), shard, blocks)

    res["peer_ldst_ms"] = timed(run_peer, iters, flush, world)
    res["nccl_ms"] = timed(lambda: tdist.all_gather_into_tensor(gathered, mine), iters, flush, world)
    roof_ms = (world - 1) * shard / (NVLINK_GBS * 1e9) * 1e3
    res["roofline_ms"] = roof_ms
    res["peer_ldst_frac_of_roofline"] = roof_ms / res["peer_ldst_ms"]
    res["nccl_frac_of_roofline"] = roof_ms / res["nccl_ms"]
    res["inbound_gbs_ldst"] = (world - 1) * shard / res["peer_ldst_ms"] / 1e6
    assert lib.ft_gemm_error() == 0
    symm.close()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", nargs="+", default=["rs", "ag"], help="rs, ag, gather")
    ap.add_argument("--gather-mib", nargs="+", type=int, default=[605, 1632],
                    help="unit sizes of the gather benchmark (13B and 70B layers in bf16)")
    ap.add_argument("--sizes", nargs="+", default=["1M", "16M", "256M", "1B"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--blocks", type=int, default=148)
    args = ap.parse_args()
    ft.init_distributed("nccl")
    world, rank = ft.distributed.get_world_size(), ft.distributed.get_rank()
    dev = ft.distributed.current_device()
    page = FlagPage()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    out = []
    if "rs" in args.what:
        for name in args.sizes:
            out.append(bench_rs(world, rank, dev, page, SIZES[name], args.iters, flush, args.blocks))
    if "gather" in args.what:
        for mib in args.gather_mib:
            out.append(bench_gather(world, rank, dev, page, mib << 20, args.iters, flush, args.blocks))
    if "ag" in args.what:
        out.append(bench_ag(world, rank, dev, page, args.iters, flush))
    if rank == 0:
        for r in out:
            print(json.dumps(r), flush=True)
    tdist.barrier()
    page.close()
    tdist.destroy_process_group()


if __name__ == "__main__":
    main()
