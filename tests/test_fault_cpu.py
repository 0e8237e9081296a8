"""Failure detection without touching a GPU: a gloo rank raises in the middle of
a step; the other rank must come back with an error that names the failed peer
within the (short) process-group timeout instead of hanging, and a slow step
must trip the watchdog."""
import os
import time
from datetime import timedelta

import pytest

import torch
import torch.multiprocessing as mp


def _worker(rank, world, port, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(1)
    import flextrain_b200 as ft
    from flextrain_b200.models.llama import preset
    from flextrain_b200.testing import build_llama_engine
    from flextrain_b200.utils.health import PeerFailure
    ft.init_distributed("gloo", timeout=timedelta(seconds=8))
    cfg = preset("tiny", num_layers=2, hidden=64, num_heads=2, ffn=128, vocab=128, seq_len=16)
    tok = torch.randint(0, 128, (1, 17))
    calls = {"n": 0}

    def batch_fn():
        calls["n"] += 1
        if rank == 1 and calls["n"] == 3:
            raise RuntimeError("injected failure on rank 1")
        return tok[:, :-1], tok[:, 1:]

    ft_cfg = {"batch_size": 2, "micro_batch_size": 1, "mixed_precision": {"device_dtype": "fp32"}}
    model, opt, eng = build_llama_engine(cfg, ft_cfg, batch_fn)
    t0 = time.time()
    outcome = "finished"
    try:
        for _ in range(5):
            eng.train_iteration()
    except PeerFailure as e:
        outcome = f"peer:{e}"
    except RuntimeError as e:
        outcome = f"own:{e}" if "injected" in str(e) else f"runtime:{e}"
    q.put((rank, outcome, time.time() - t0, eng.global_steps))
    q.close()
    q.join_thread()                                   # flush before the hard exit below
    os._exit(0 if outcome == "finished" else 3)       # no orderly teardown with a dead peer


def test_failed_rank_is_reported_not_waited_for():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29800 + os.getpid() % 150
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict()
    for _ in procs:
        rank, outcome, secs, steps = q.get(timeout=120)
        got[rank] = (outcome, secs, steps)
    for p in procs:
        p.join(30)
        assert p.exitcode == 3
    assert got[1][0].startswith("own:") and got[1][2] == 2
    assert got[0][0].startswith("peer:") and "rank 1 failed" in got[0][0] and "injected" in got[0][0]
    assert got[0][1] < 60


def test_watchdog_trips_on_a_slow_step(fresh_runtime):
    from flextrain_b200.models.llama import preset
    from flextrain_b200.testing import build_llama_engine
    cfg = preset("tiny", num_layers=2, hidden=64, num_heads=2, ffn=128, vocab=128, seq_len=16)
    tok = torch.randint(0, 128, (2, 17))
    slow = {"on": False}

    def batch_fn():
        if slow["on"]:
            time.sleep(1.2)
        return tok[:, :-1], tok[:, 1:]

    ft_cfg = {"batch_size": 2, "micro_batch_size": 2, "mixed_precision": {"device_dtype": "fp32"},
              "engine": {"watchdog_seconds": 0.5}}
    model, opt, eng = build_llama_engine(cfg, ft_cfg, batch_fn, backend="gloo")
    eng.train_iteration()                     # first step pays one-off costs
    eng.watchdog.reset()
    eng.train_iteration()
    assert not eng.health()["watchdog_tripped"]
    slow["on"] = True
    eng.train_iteration()
    assert eng.health()["watchdog_tripped"]
    eng.shutdown()


def _fallback_worker(rank, world, port, q):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(1)
    import flextrain_b200 as ft
    from flextrain_b200.models.llama import preset
    from flextrain_b200.testing import build_llama_engine, reset_runtime
    ft.init_distributed("gloo")
    cfg = preset("tiny", num_layers=2, hidden=64, num_heads=2, ffn=128, vocab=128, seq_len=16)
    tok = torch.randint(0, 128, (1, 17))
    ft_cfg = {"batch_size": 2, "micro_batch_size": 1, "mixed_precision": {"device_dtype": "fp32"}}
    model, opt, eng = build_llama_engine(cfg, ft_cfg, lambda: (tok[:, :-1], tok[:, 1:]))
    # pretend the peer-memory kernels are in use, then report a wait that ran out on ONE rank only
    eng.opts._fused = True
    eng.para._peer_gather = True
    eng._fused_health_check(read_words=lambda: (0, 0))
    clean = (eng.opts._fused, eng.para._peer_gather)
    eng._fused_health_check(read_words=lambda: (7, 0))          # a GEMM-internal code is kept, not a time-out
    kept = eng.health().get("gemm_error_word_seen")
    eng._fused_health_check(read_words=lambda: (0, 101) if rank == 1 else (0, 0))
    after = (eng.opts._fused, eng.para._peer_gather, eng.health().get("fused_collectives_disabled"))
    # at the end of a step the same finding is an error on EVERY rank (the step is incomplete) ...
    from flextrain_b200.utils.health import FusedCollectiveTimeout
    eng.opts._fused = True
    skipped = eng.skipped_steps
    try:
        eng._fused_health_check(read_words=lambda: (0, 101) if rank == 1 else (0, 0), end_of_step=True)
        raised = False
    except FusedCollectiveTimeout:
        raised = True
    counted = eng.skipped_steps == skipped + 1 and not eng.opts._fused
    # ... unless the configuration asks for a silent switch
    eng.config.engine.fused_timeout_action = "fallback"
    eng.opts._fused = True
    eng._fused_health_check(read_words=lambda: (201, 0) if rank == 0 else (0, 0), end_of_step=True)
    quiet = not eng.opts._fused
    loss = float(eng.train_iteration()[0].detach())             # and the run goes on, on the library collectives
    eng.shutdown()
    q.put((rank, clean, kept, after + (raised, counted, quiet), loss))
    reset_runtime()


def test_timeout_on_one_rank_switches_every_rank_to_library_collectives():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29950 + os.getpid() % 40
    procs = [ctx.Process(target=_fallback_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = {}
    for _ in procs:
        rank, clean, kept, after, loss = q.get(timeout=120)
        got[rank] = (clean, kept, after, loss)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank in (0, 1):
        clean, kept, after, loss = got[rank]
        assert clean == (True, True)                    # no time-out: nothing changes
        assert kept == 7
        assert after == (False, False, True, True, True, True), f"rank {rank} did not switch: {after}"
        assert loss == loss


@pytest.mark.parametrize("kind", ["eio", "short"])
def test_nvme_fault_during_a_step_surfaces_and_leaves_nothing_in_flight(kind, fresh_runtime, tmp_path):
    """A block transfer that fails while the engine trains over NVMe tiers: the step ends
    with an exception that names the I/O error (whether the main thread or a background
    update met it), no request stays in flight and the engine shuts down without waiting
    for anything."""
    import torch
    from flextrain_b200.memory.nvme_swapper import NVMeError, get_nvme_swapper
    from flextrain_b200.models.llama import preset
    from flextrain_b200.testing import build_llama_engine
    cfg = preset("tiny", num_layers=4, hidden=64, num_heads=2, ffn=136, vocab=128, seq_len=16)
    gen = torch.Generator().manual_seed(5)
    data = torch.randint(0, 128, (2, 17), generator=gen)
    split = {"parameter": [0.0, 0.5], "optimizer": [0.0, 0.5], "checkpoint": [0.0, 0.5], "gradient": [0.0, 1.0]}
    ft_cfg = {"batch_size": 2, "micro_batch_size": 2, "mixed_precision": {"device_dtype": "fp32"},
              "split_ratio": split, "nvme_swap": {"swap_dir": str(tmp_path), "aio_thread_count": 1}}
    model, opt, eng = build_llama_engine(cfg, ft_cfg, lambda: (data[:, :-1].contiguous(), data[:, 1:].contiguous()),
                                         lr=1e-3, backend="gloo")
    eng.train_iteration()                                   # a clean step first
    eng.synchronize()
    swapper = get_nvme_swapper()
    swapper.engine.inject_fault(kind, 1)
    with pytest.raises(Exception) as info:
        eng.train_iteration()
        eng.synchronize()
    chain, exc = [], info.value
    while exc is not None:
        chain.append(exc)
        exc = exc.__cause__ or exc.__context__
    assert any(isinstance(e, NVMeError) for e in chain), [repr(e) for e in chain]
    assert swapper.engine.pending() == 0
    eng.shutdown()
