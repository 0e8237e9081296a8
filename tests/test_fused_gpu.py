"""Fused reduce-scatter + unscale + Adam kernel on ONE GPU.

Several ranks cannot be run as separate waiting kernels on one device, so the
ranks are emulated: all "peer" buffers live on this GPU and every flag word is
set to the call's sequence number beforehand, which makes both barriers pass at
once.  What is checked is the math: the slice owner's sum over ranks, the
unscale, Adam on the HBM share against the host kernel, and the gradient
hand-off of the host share."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


class _Owner:
    defaults = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, bias_correction=True)
    adamw_mode = True


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("gdt", [torch.bfloat16, torch.float32])
def test_rs_adam_emulated_ranks(world, gdt):
    from flextrain_b200.ops.adam.cpu_adam import cpu_adam_update
    from flextrain_b200.parallel import fused
    from flextrain_b200.param_group import GroupSegment
    dev = torch.device("cuda", 0)
    torch.manual_seed(world)
    S, og, a_hi = 8 * 4099, 8 * 2048, 8 * 1000
    grads = [(torch.randn(world * S, device=dev) * 8).to(gdt) for _ in range(world)]
    flags = [torch.zeros(128 * 8, dtype=torch.int32, device=dev) for _ in range(world)]
    seq = 3
    for f in flags:
        f.fill_(seq)
    loss_scale = 16.0
    groups = [dict(weight_decay=0.01), dict(weight_decay=0.0, lr=5e-4)]
    segs = [GroupSegment(0, 0, 8 * 1500), GroupSegment(1, 8 * 1500, og)]
    for rank in range(world):
        master = torch.randn(og, device=dev)
        m, v = torch.rand(og, device=dev) * 0.1, torch.rand(og, device=dev) * 0.1
        ref_master, ref_m, ref_v = master.cpu().clone(), m.cpu().clone(), v.cpu().clone()
        param_a = torch.zeros(a_hi, device=dev, dtype=torch.bfloat16)
        param_b = torch.zeros(og - a_hi, device=dev, dtype=torch.bfloat16)
        host_grad = torch.zeros(S - og, dtype=gdt).pin_memory()
        flag = torch.zeros(1, dtype=torch.int32, device=dev)
        gp = (ctypes.c_void_p * world)(*[g.data_ptr() for g in grads])
        fp = (ctypes.c_void_p * world)(*[f.data_ptr() for f in flags])
        arr = fused.make_segments(segs, groups, _Owner, step=2)
        fused.rs_adam(world, rank, gp, fp, gdt, S, 1.0 / (world * loss_scale), seq, None, og, True,
                      master, m, v, param_a, a_hi, param_b, torch.bfloat16, host_grad, flag, arr,
                      len(segs), max_blocks=16)
        torch.cuda.synchronize()
        assert fused.comm_error() == 0
        want = sum(g[rank * S:(rank + 1) * S].float() for g in grads) / (world * loss_scale)
        want = want.cpu()
        assert torch.allclose(host_grad.float(), want[og:].to(gdt).float(), rtol=1e-2, atol=1e-3)
        for seg in segs:
            grp = {**_Owner.defaults, **groups[seg.group]}
            sl = slice(seg.start, seg.end)
            cpu_adam_update(2, grp["lr"], 0.9, 0.999, 1e-8, grp["weight_decay"], True, True,
                            ref_master[sl], want[sl].contiguous(), ref_m[sl], ref_v[sl])
        assert torch.allclose(master.cpu(), ref_master, rtol=1e-5, atol=1e-6)
        assert torch.allclose(m.cpu(), ref_m, rtol=1e-5, atol=1e-7)
        assert torch.allclose(v.cpu(), ref_v, rtol=1e-5, atol=1e-7)
        out = torch.cat([param_a, param_b]).cpu().float()
        assert torch.allclose(out, ref_master.to(torch.bfloat16).float(), rtol=1e-2, atol=1e-3)
        assert flag.item() == 0


def test_rs_adam_two_phase_and_overflow_flag():
    from flextrain_b200.parallel import fused
    dev = torch.device("cuda", 0)
    world, S = 2, 8 * 512
    grads = [torch.randn(world * S, device=dev).to(torch.float16) for _ in range(world)]
    grads[1][S + 17] = float("inf")          # inside rank 1's slice
    flags = [torch.full((128 * 8,), 1, dtype=torch.int32, device=dev) for _ in range(world)]
    gp = (ctypes.c_void_p * world)(*[g.data_ptr() for g in grads])
    fp = (ctypes.c_void_p * world)(*[f.data_ptr() for f in flags])
    for rank, expect in ((0, 0), (1, 1)):
        flag = torch.zeros(1, dtype=torch.int32, device=dev)
        want = sum(g[rank * S:(rank + 1) * S].float() for g in grads) / world
        reduced = grads[rank][rank * S:(rank + 1) * S]
        fused.rs_adam(world, rank, gp, fp, torch.float16, S, 1.0 / world, 1, reduced, 0, False, None,
                      None, None, None, 0, None, torch.float16, None, flag,
                      fused.make_segments([], [], None, 1) if False else (fused._AdamSegment * 1)(), 0)
        torch.cuda.synchronize()
        assert flag.item() == expect
        if not expect:
            assert torch.allclose(reduced.float(), want.to(torch.float16).float(), rtol=1e-2, atol=1e-2)


def test_bounded_wait_reports_instead_of_hanging():
    """A start flag that nobody sets: the kernel must give up, raise the error
    word, report through the caller's status word, leave every output (fp32
    state, parameters, host gradient) untouched and leave the context usable
    (checked by running another kernel)."""
    import os
    from flextrain_b200.parallel import fused
    from flextrain_b200.param_group import GroupSegment
    dev = torch.device("cuda", 0)
    if os.environ.get("FLEXTRAIN_SKIP_TIMEOUT_TEST"):
        pytest.skip("disabled by environment")
    world, S, og = 2, 8 * 64, 8 * 32
    grads = [torch.randn(world * S, device=dev).to(torch.bfloat16) for _ in range(world)]
    flags = [torch.zeros(128 * 8, dtype=torch.int32, device=dev) for _ in range(world)]
    gp = (ctypes.c_void_p * world)(*[g.data_ptr() for g in grads])
    fp = (ctypes.c_void_p * world)(*[f.data_ptr() for f in flags])
    master = torch.randn(og, device=dev)
    m, v = torch.rand(og, device=dev), torch.rand(og, device=dev)
    param = torch.full((og,), 3.0, device=dev, dtype=torch.bfloat16)
    host_grad = torch.full((S - og,), 7.0, dtype=torch.bfloat16).pin_memory()
    status = torch.zeros(1, dtype=torch.int32).pin_memory()
    before = [t.clone() for t in (master, m, v, param)]
    arr = fused.make_segments([GroupSegment(0, 0, og)], [dict()], _Owner, step=1)
    from flextrain_b200.ops.native import cuda_lib
    lib = cuda_lib()
    lib.ft_comm_set_spin_budget.argtypes = [ctypes.c_longlong]
    lib.ft_comm_set_spin_budget(20_000_000)          # ~10 ms
    try:
        fused.rs_adam(world, 0, gp, fp, torch.bfloat16, S, 0.5, 7, None, og, True, master, m, v,
                      param, og, None, torch.bfloat16, host_grad, None, arr, 1, max_blocks=2,
                      status=status)
        torch.cuda.synchronize()
        assert fused.comm_error() == 101
    finally:
        lib.ft_comm_set_spin_budget(0)
    assert int(status.item()) == 101
    for now, was in zip((master, m, v, param), before):
        assert torch.equal(now, was)
    assert torch.equal(host_grad, torch.full_like(host_grad, 7.0))
    x = torch.ones(1024, device=dev)
    assert float((x * 2).sum()) == 2048.0


@pytest.mark.parametrize("world", [1, 2, 4])
def test_ag_gemm_emulated_ranks(world):
    """All ranks' weight buffers on one GPU, barriers pre-satisfied: the copy warps
    pull the 'remote' row shards while the tensor cores multiply."""
    from flextrain_b200.ops.native import cuda_lib
    from flextrain_b200.parallel import fused
    dev = torch.device("cuda", 0)
    torch.manual_seed(7)
    M, N, K = 512, 256 * world * 2, 320
    W = (torch.randn(N, K, device=dev) * 0.1).to(torch.bfloat16)
    x = torch.randn(M, K, device=dev).to(torch.bfloat16)
    rows = N // world
    bufs = []
    for r in range(world):
        b = torch.zeros(N, K, device=dev, dtype=torch.bfloat16)
        b[r * rows:(r + 1) * rows] = W[r * rows:(r + 1) * rows]     # only the own shard is in place
        bufs.append(b)
    flags = [torch.full((128 * 8,), 5, dtype=torch.int32, device=dev) for _ in range(world)]
    wp = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])
    fp = (ctypes.c_void_p * world)(*[f.data_ptr() for f in flags])
    want = x.float() @ W.float().t()
    for rank in range(world):
        y = fused.ag_gemm(world, rank, wp, fp, 5, x, N)
        torch.cuda.synchronize()
        assert cuda_lib().ft_gemm_error() == 0
        err = ((y.float() - want).norm() / want.norm()).item()
        assert err < 1e-2, f"rank {rank}: {err}"
        assert torch.equal(bufs[rank], W), "the local buffer must hold the whole weight afterwards"


@pytest.mark.parametrize("world,w_off_chunks,n", [(2, 0, 520), (4, 3, 1000), (8, 5, 300), (8, 0, 1536), (3, 40, 264)])
def test_ag_gemm_window_of_a_flat_sharded_buffer(world, w_off_chunks, n):
    """The weight is a window of a larger flat buffer that the ranks shard in contiguous
    pieces, as the engine keeps a layer: ownership boundaries fall anywhere in the matrix
    (inside a 256-row block, some ranks own nothing of it), rows are not a multiple of 256."""
    from flextrain_b200.ops.native import cuda_lib
    from flextrain_b200.parallel import fused
    dev = torch.device("cuda", 0)
    torch.manual_seed(world * 100 + n)
    M, K = 384, 256
    chunk = fused.AG_GEMM_CHUNK
    w_off = w_off_chunks * chunk
    w_bytes = n * K * 2
    total = w_off + w_bytes + 7 * chunk                      # other parameters follow the matrix
    shard = -(-total // (world * chunk)) * chunk              # contiguous pieces, chunk-aligned
    full = torch.randint(0, 255, (shard * world,), dtype=torch.uint8, device=dev)
    Wm = (torch.randn(n, K, device=dev) * 0.1).to(torch.bfloat16)
    full[w_off:w_off + w_bytes] = Wm.view(torch.uint8).reshape(-1)
    x = torch.randn(M, K, device=dev).to(torch.bfloat16)
    want = x.float() @ Wm.float().t()
    bufs = []
    for r in range(world):
        b = torch.full((shard * world,), 0, dtype=torch.uint8, device=dev)
        b[r * shard:(r + 1) * shard] = full[r * shard:(r + 1) * shard]
        bufs.append(b)
    flags = [torch.full((128 * 8,), 2, dtype=torch.int32, device=dev) for _ in range(world)]
    bp = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])
    fp = (ctypes.c_void_p * world)(*[f.data_ptr() for f in flags])
    for rank in range(world):
        before = bufs[rank].clone()
        y = fused.ag_gemm(world, rank, bp, fp, 2, x, n, w_off_bytes=w_off, shard_bytes=shard)
        torch.cuda.synchronize()
        assert cuda_lib().ft_gemm_error() == 0
        err = ((y.float() - want).norm() / want.norm()).item()
        assert err < 1e-2, f"rank {rank}: {err}"
        got = bufs[rank]
        assert torch.equal(got[w_off:w_off + w_bytes], full[w_off:w_off + w_bytes])
        # nothing outside the window was touched
        assert torch.equal(got[:w_off], before[:w_off]) and torch.equal(got[w_off + w_bytes:], before[w_off + w_bytes:])
        bufs[rank].copy_(before)                              # the next emulated rank's peers own only their shards


@pytest.mark.parametrize("world,lo_chunks,hi_chunks", [(4, 0, 0), (4, 3, 9), (8, 1, 2), (2, 0, 5)])
def test_peer_gather_range_emulated_ranks(world, lo_chunks, hi_chunks):
    """Gather of a byte range of the flat buffer: everything outside the range and everything
    this rank owns stay as they were."""
    from flextrain_b200.ops.native import cuda_lib
    from flextrain_b200.parallel import fused
    dev = torch.device("cuda", 0)
    shard = 4096 * 5
    total = shard * world
    lo, hi = lo_chunks * 4096 + 16 * 3, total - hi_chunks * 4096 - 16 * 5
    full = torch.randint(1, 255, (total,), dtype=torch.uint8, device=dev)
    bufs = []
    for r in range(world):
        b = torch.zeros(total, dtype=torch.uint8, device=dev)
        b[r * shard:(r + 1) * shard] = full[r * shard:(r + 1) * shard]
        bufs.append(b)
    flags = [torch.full((128 * 8,), 4, dtype=torch.int32, device=dev) for _ in range(world)]
    bp = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])
    fp = (ctypes.c_void_p * world)(*[f.data_ptr() for f in flags])
    rank = world - 1
    fused.peer_gather_range(world, rank, bp, fp, 4, shard, lo, hi, num_copiers=5)
    torch.cuda.synchronize()
    assert cuda_lib().ft_gemm_error() == 0
    want = torch.zeros(total, dtype=torch.uint8, device=dev)
    want[rank * shard:(rank + 1) * shard] = full[rank * shard:(rank + 1) * shard]
    want[lo:hi] = full[lo:hi]
    assert torch.equal(bufs[rank], want)


def test_peer_gather_emulated_ranks():
    from flextrain_b200.ops.native import cuda_lib
    from flextrain_b200.parallel import fused
    dev = torch.device("cuda", 0)
    world = 4
    shard = 4096 * 37 + 4096                      # bytes, page aligned, not a multiple of 32 KiB
    full = torch.randint(0, 255, (world * shard,), dtype=torch.uint8, device=dev)
    bufs = []
    for r in range(world):
        b = torch.zeros(world * shard, dtype=torch.uint8, device=dev)
        b[r * shard:(r + 1) * shard] = full[r * shard:(r + 1) * shard]
        bufs.append(b)
    flags = [torch.full((128 * 8,), 9, dtype=torch.int32, device=dev) for _ in range(world)]
    bp = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])
    fp = (ctypes.c_void_p * world)(*[f.data_ptr() for f in flags])
    fused.peer_gather(world, 2, bp, fp, 9, shard, num_copiers=3)
    torch.cuda.synchronize()
    assert cuda_lib().ft_gemm_error() == 0
    assert torch.equal(bufs[2], full)


@pytest.mark.parametrize("world", [1, 2, 8])
def test_ar_adam_emulated_ranks(world):
    """All-reduce form: every emulated rank reduces its slice, updates its slice
    of the state and stores the new parameters into all ranks' buffers; after
    all ranks ran, every buffer holds the whole updated vector."""
    from flextrain_b200.ops.adam.cpu_adam import cpu_adam_update
    from flextrain_b200.parallel import fused
    from flextrain_b200.param_group import GroupSegment, slice_segments
    dev = torch.device("cuda", 0)
    torch.manual_seed(10 + world)
    S = 8 * 1031
    N = world * S
    grads = [(torch.randn(N, device=dev) * 4).to(torch.bfloat16) for _ in range(world)]
    paras = [torch.zeros(N, device=dev, dtype=torch.bfloat16) for _ in range(world)]
    flags = [torch.full((128 * 8,), 5, dtype=torch.int32, device=dev) for _ in range(world)]
    gp = (ctypes.c_void_p * world)(*[g.data_ptr() for g in grads])
    pp = (ctypes.c_void_p * world)(*[p.data_ptr() for p in paras])
    fp = (ctypes.c_void_p * world)(*[f.data_ptr() for f in flags])
    groups = [dict(weight_decay=0.01), dict(weight_decay=0.0, lr=5e-4)]
    cut = 8 * 700
    global_segs = [GroupSegment(0, 0, cut), GroupSegment(1, cut, N)]
    master0 = torch.randn(N)
    ref_master, ref_m, ref_v = master0.clone(), torch.zeros(N), torch.zeros(N)
    want = (sum(g.float() for g in grads) / (world * 4.0)).cpu()
    for seg in global_segs:
        grp = {**_Owner.defaults, **groups[seg.group]}
        sl = slice(seg.start, seg.end)
        cpu_adam_update(1, grp["lr"], 0.9, 0.999, 1e-8, grp["weight_decay"], True, True,
                        ref_master[sl], want[sl].contiguous(), ref_m[sl], ref_v[sl])
    for rank in range(world):
        lo = rank * S
        segs = slice_segments(global_segs, lo, lo + S, rebase=True)
        master = master0[lo:lo + S].to(dev)
        m, v = torch.zeros(S, device=dev), torch.zeros(S, device=dev)
        arr = fused.make_segments(segs, groups, _Owner, step=1)
        fused.ar_adam(world, rank, gp, fp, torch.bfloat16, S, 1.0 / (world * 4.0), 5, None, True,
                      master, m, v, pp, torch.bfloat16, None, arr, len(segs), max_blocks=16)
        torch.cuda.synchronize()
        assert fused.comm_error() == 0
        assert torch.allclose(master.cpu(), ref_master[lo:lo + S], rtol=1e-5, atol=1e-6)
        assert torch.allclose(v.cpu(), ref_v[lo:lo + S], rtol=1e-5, atol=1e-7)
    for p in paras:
        assert torch.allclose(p.cpu().float(), ref_master.to(torch.bfloat16).float(), rtol=1e-2, atol=1e-3)
