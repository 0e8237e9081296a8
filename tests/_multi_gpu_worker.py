"""Worker launched by tests/test_fused_multi_gpu.py under torch.distributed.run
(one process per GPU, NCCL).  Exits non-zero on any mismatch."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def case_rs_adam():
    import ctypes
    import torch.distributed as tdist
    import flextrain_b200 as ft
    from flextrain_b200.parallel import fused
    from flextrain_b200.parallel.symm_mem import FlagPage, SymmetricBuffer
    from flextrain_b200.param_group import GroupSegment
    ft.init_distributed("nccl")
    world, rank = ft.distributed.get_world_size(), ft.distributed.get_rank()
    dev = ft.distributed.current_device()

    class Owner:
        defaults = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, bias_correction=True)
        adamw_mode = True

    S = 8 * 100_000
    og = 8 * 60_000
    page = FlagPage()
    for gdt in (torch.bfloat16, torch.float32):
        symm = SymmetricBuffer(world * S * torch.empty((), dtype=gdt).element_size())
        for it in range(3):
            torch.manual_seed(100 * it + rank)
            mine = symm.tensor(gdt)
            mine.copy_((torch.randn(world * S, device=dev) * 4).to(gdt))
            ref_full = mine.float().clone()
            tdist.all_reduce(ref_full)
            want = ref_full[rank * S:(rank + 1) * S] / (world * 8.0)
            master = torch.zeros(og, device=dev)
            m, v = torch.zeros(og, device=dev), torch.zeros(og, device=dev)
            out = torch.zeros(og, device=dev, dtype=torch.bfloat16)
            host = torch.zeros(S - og, dtype=gdt).pin_memory()
            segs = [GroupSegment(0, 0, og)]
            torch.cuda.synchronize()
            tdist.barrier()
            fused.rs_adam(world, rank, symm.ptr_array(), page.ptr_array(), gdt, S, 1.0 / (world * 8.0),
                          page.next_seq("t"), None, og, True, master, m, v, out, og, None, torch.bfloat16,
                          host, None, fused.make_segments(segs, [{}], Owner, 1), 1, max_blocks=32)
            torch.cuda.synchronize()
            assert fused.comm_error() == 0
            tol = 2e-2 if gdt == torch.bfloat16 else 1e-5
            assert torch.allclose(host.float().to(dev), want[og:], rtol=tol, atol=tol), "host grads"
            # first Adam step from zero state: m = (1 - beta1) * g is linear in the reduced
            # gradient; p = -lr * g / (|g| + eps) is checked away from g = 0, where the order of
            # the fp32 sum over more than two ranks decides its sign
            g = want[:og]
            assert torch.allclose(m / 0.1, g, rtol=tol, atol=tol), "adam first moment"
            expect = -1e-3 * g / (g.abs() + 1e-8)
            big = g.abs() > 1e-2
            assert torch.allclose(master[big], expect[big], rtol=1e-3, atol=1e-6), "adam"
            tdist.barrier()
        symm.close()
    page.close()
    print(f"rank {rank}: rs_adam ok", flush=True)


def case_engine(fused_mode: bool):
    """Four steps of the tiny Llama with the library collectives or with the fused kernels;
    rank 0 writes the losses to the file named by FT_TEST_LOSSES (the two modes run as two
    launches: one process group per process keeps NCCL's bootstrap out of the comparison)."""
    import json
    import flextrain_b200 as ft
    from flextrain_b200.models.llama import preset
    from flextrain_b200.testing import build_llama_engine
    ft.init_distributed("nccl")
    world, rank = ft.distributed.get_world_size(), ft.distributed.get_rank()
    dev = ft.distributed.current_device()
    cfg = preset("tiny", num_layers=4, hidden=256, num_heads=4, ffn=768, vocab=1024, seq_len=256)
    gen = torch.Generator().manual_seed(1 + rank)
    data = [torch.randint(0, cfg.vocab, (2, cfg.seq_len + 1), generator=gen).to(dev) for _ in range(2)]
    it = {"i": 0}

    def batch_fn():
        t = data[it["i"] % 2]
        it["i"] += 1
        return t[:, :-1], t[:, 1:]

    ft_cfg = {"batch_size": 4 * world, "micro_batch_size": 2,
              "mixed_precision": {"device_dtype": "bf16", "dynamic_loss_scaling": False},
              "split_ratio": {"parameter": [0.5, 0.5], "optimizer": [0.5, 0.5],
                              "checkpoint": [1.0, 0.0], "gradient": [1.0, 0.0]},
              "engine": {"fused_collectives": fused_mode, "num_unit_buffers": 3}}
    model, opt, eng = build_llama_engine(cfg, ft_cfg, batch_fn, lr=1e-3, init_device=dev,
                                         dtype=torch.bfloat16)
    assert eng.opts._fused == fused_mode
    assert eng.para._peer_gather == fused_mode
    losses = []
    for _ in range(4):
        r = eng.train_iteration()
        losses.append(sum(float(x.detach()) for x in r) / len(r))
    eng.synchronize()
    used = eng.collectives_in_use()
    health = eng.health()
    eng.shutdown()
    assert losses[-1] < losses[0]
    if fused_mode:
        from flextrain_b200.parallel.fused import comm_error
        assert comm_error() == 0 and not health.get("fused_collectives_disabled", False)
        assert "ft_ag_gemm" in used["first_gemm"] and "ft_rs_adam" in used["unit_reduce"], used
        assert "ft_ar_adam" in used["non_layerwise"], used
    # the mean over ranks is what both modes must agree on
    mean = [ft.distributed.all_reduce_scalar(x) / world for x in losses]
    if rank == 0:
        with open(os.environ["FT_TEST_LOSSES"], "w") as f:
            json.dump({"losses": mean, "collectives": used}, f)
    print(f"engine fused={fused_mode}: {mean}", flush=True)


def case_ag_gemm():
    import torch.distributed as tdist
    import flextrain_b200 as ft
    from flextrain_b200.ops.native import cuda_lib
    from flextrain_b200.parallel import fused
    from flextrain_b200.parallel.symm_mem import FlagPage, SymmetricBuffer
    ft.init_distributed("nccl")
    world, rank = ft.distributed.get_world_size(), ft.distributed.get_rank()
    dev = ft.distributed.current_device()
    page = FlagPage()
    M, N, K = 1024, 256 * world * 3, 512
    torch.manual_seed(3)
    full = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16)
    x = torch.randn(M, K, device=dev).to(torch.bfloat16)
    rows = N // world
    symm = SymmetricBuffer(N * K * 2)
    w = symm.tensor(torch.bfloat16).view(N, K)
    want = x.float() @ full.float().t()
    for it in range(3):
        w.zero_()
        w[rank * rows:(rank + 1) * rows].copy_(full[rank * rows:(rank + 1) * rows])
        torch.cuda.synchronize()
        tdist.barrier()
        y = fused.ag_gemm(world, rank, symm.ptr_array(), page.ptr_array(), page.next_seq("ag"), x, N)
        torch.cuda.synchronize()
        assert cuda_lib().ft_gemm_error() == 0
        assert ((y.float() - want).norm() / want.norm()).item() < 1e-2
        assert torch.equal(w, full)
        tdist.barrier()
    # whole-buffer peer gather
    flat = symm.tensor(torch.uint8)
    shard = symm.nbytes // world
    ref = torch.arange(symm.nbytes, device=dev, dtype=torch.int64).remainder_(251).to(torch.uint8)
    flat.zero_()
    flat[rank * shard:(rank + 1) * shard].copy_(ref[rank * shard:(rank + 1) * shard])
    torch.cuda.synchronize()
    tdist.barrier()
    fused.peer_gather(world, rank, symm.ptr_array(), page.ptr_array(), page.next_seq("pg"), shard, 8)
    torch.cuda.synchronize()
    assert cuda_lib().ft_gemm_error() == 0
    assert torch.equal(flat, ref)
    tdist.barrier()
    symm.close()
    page.close()
    print(f"rank {rank}: ag_gemm ok", flush=True)


if __name__ == "__main__":
    {"rs_adam": case_rs_adam, "engine_nccl": lambda: case_engine(False),
     "engine_fused": lambda: case_engine(True), "ag_gemm": case_ag_gemm}[sys.argv[1]]()
    if torch.distributed.is_initialized():
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
