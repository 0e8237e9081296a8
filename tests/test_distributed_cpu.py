"""The gloo backend of the distributed wrapper: emulated reduce-scatter / AVG."""
import os

import torch
import torch.multiprocessing as mp


def _worker(rank, world, port, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    from flextrain_b200.utils import distributed as dist
    dist.init_distributed("gloo")
    assert dist.get_world_size() == world and dist.get_rank() == rank
    assert dist.current_device().type == "cpu" and dist.get_backend() == "gloo"
    full = torch.arange(world * 4, dtype=torch.float32) * (rank + 1)
    out = torch.empty(4)
    dist.reduce_scatter(out, full, dist.ReduceOp.AVG)
    want = torch.arange(world * 4, dtype=torch.float32)[rank * 4:(rank + 1) * 4] * (sum(range(1, world + 1)) / world)
    ok = torch.allclose(out, want)
    inplace = full.clone()
    h = dist.reduce_scatter(inplace[rank * 4:(rank + 1) * 4], inplace, dist.ReduceOp.SUM, async_op=True)
    h.wait()
    ok &= torch.allclose(inplace[rank * 4:(rank + 1) * 4], want * world)
    t = torch.full((3,), float(rank))
    dist.all_reduce(t, dist.ReduceOp.AVG)
    ok &= torch.allclose(t, torch.full((3,), (world - 1) / 2))
    gathered = torch.empty(world * 2)
    dist.all_gather(gathered, torch.full((2,), float(rank)))
    ok &= torch.equal(gathered, torch.arange(world).repeat_interleave(2).float())
    b = torch.full((2,), float(rank))
    dist.broadcast(b, src=1)
    ok &= torch.equal(b, torch.ones(2))
    ok &= dist.all_reduce_scalar(1.0) == world
    dist.barrier()
    dist.shutdown()
    q.put(bool(ok))


def test_gloo_world_3():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + os.getpid() % 200
    procs = [ctx.Process(target=_worker, args=(r, 3, port, q)) for r in range(3)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(60)
    assert all(results)


def test_world_size_one_needs_no_process_group():
    from flextrain_b200.utils import distributed as dist
    dist.shutdown()
    os.environ.pop("WORLD_SIZE", None)
    dist.init_distributed("gloo", force_init=False)
    assert dist.get_world_size() == 1 and not torch.distributed.is_initialized()
    x = torch.arange(4.)
    out = torch.empty(4)
    assert dist.reduce_scatter(out, x).is_completed() and torch.equal(out, x)
    assert dist.all_reduce(x).is_completed()
    dist.barrier()
    dist.shutdown()


def _sub_group_worker(rank, world, port, q):
    import os
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as tdist
    from flextrain_b200.utils import distributed as dist
    dist.init_distributed(dist_backend="gloo")
    pair = tdist.new_group([0, 1])                       # every rank creates it, ranks 0 and 1 use it
    out = None
    if rank < 2:
        t = torch.full((4,), float(rank + 1))
        dist.all_reduce(t, dist.ReduceOp.AVG, pair)       # the reference's order: (tensor, op, group, async_op)
        full = torch.arange(4.0) + rank
        piece = torch.empty(2)
        dist.reduce_scatter(piece, full, dist.ReduceOp.SUM, group=pair)
        out = (t.tolist(), piece.tolist())
    dist.barrier()
    q.put((rank, out))
    dist.shutdown()


def test_collectives_accept_a_group_in_the_reference_position():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 400) + 17
    procs = [ctx.Process(target=_sub_group_worker, args=(r, 3, port, q)) for r in range(3)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=120) for _ in range(3))
    for p in procs:
        p.join(timeout=60)
    assert got[0][0] == [1.5] * 4 and got[1][0] == [1.5] * 4 and got[2] is None
    assert got[0][1] == [1.0, 3.0] and got[1][1] == [5.0, 7.0]
