import os

import pytest
import torch

from flextrain_b200.config import init_flextrain_config, reset_flextrain_config
from flextrain_b200.memory import FlexTrainDataID, FlexTrainDataType
from flextrain_b200.memory.nvme_swapper import (AsyncNVMeSwapper, NVMeEngine, NVMeError, NVMeGroup,
                                                reset_nvme_swapper)


@pytest.fixture
def swap_cfg(tmp_path):
    reset_flextrain_config()
    init_flextrain_config({"batch_size": 2, "micro_batch_size": 1,
                           "nvme_swap": {"swap_dir": str(tmp_path), "aio_thread_count": 3}}, log=False)
    yield str(tmp_path)
    reset_nvme_swapper()
    reset_flextrain_config()


@pytest.mark.parametrize("engine", ["auto", "io_uring", "aio", "psync"])
@pytest.mark.parametrize("numel", [1024, 3 * 2 ** 20 + 4096, 1000])     # last: not page aligned
def test_round_trip_every_engine(tmp_path, engine, numel):
    e = NVMeEngine(block_size=1 << 20, queue_depth=4, threads=3, engine=engine)
    x = torch.randn(numel)
    y = torch.zeros_like(x)
    path = str(tmp_path / "a.swp")
    e.write(path, x)
    e.read(path, y)
    assert torch.equal(x, y)
    assert os.path.getsize(path) == numel * 4
    e.close()


def test_offsets_async_ops_and_fd_cache(tmp_path):
    e = NVMeEngine(threads=2)
    path = str(tmp_path / "b.swp")
    parts = [torch.full((4096,), float(i)) for i in range(8)]
    ids = [e.submit(path, p, True, file_offset=i * 4096 * 4) for i, p in enumerate(parts)]
    assert e.wait_all() == len(ids)
    whole = torch.empty(8 * 4096)
    e.read(path, whole)
    assert torch.equal(whole, torch.cat(parts))
    for p in parts:
        e.write(path, p)
        e.read(path, torch.empty_like(p))
    fds = e.open_fds()
    assert 2 <= fds <= 4                          # per (file, mode[, buffered]): never one per operation
    for p in parts:
        e.write(path, p)
        e.read(path, torch.empty_like(p))
    assert e.open_fds() == fds and e.pending() == 0
    assert e.forget(path) == fds and e.open_fds() == 0
    e.close()


@pytest.mark.parametrize("kind", ["eio", "short"])
def test_injected_faults_surface_as_exceptions(tmp_path, kind):
    e = NVMeEngine(threads=1, engine="psync")
    path = str(tmp_path / "c.swp")
    x = torch.randn(1 << 18)
    e.write(path, x)
    e.inject_fault(kind, 1)
    with pytest.raises(NVMeError):
        e.read(path, torch.empty_like(x))
    assert e.pending() == 0                       # nothing left in flight after the failure
    y = torch.empty_like(x)
    e.read(path, y)                               # the engine stays usable
    assert torch.equal(x, y)
    with pytest.raises(NVMeError):
        e.read(str(tmp_path / "missing.swp"), y)
    e.close()


def test_swapper_names_files_like_the_reference(swap_cfg):
    sw = AsyncNVMeSwapper()
    did = FlexTrainDataID(FlexTrainDataType.PARA, 3)
    assert str(did) == "rank0_PARA_layer3.swp"
    x = torch.randn(8192)
    sw.swap_out(did, x)
    assert os.path.exists(os.path.join(swap_cfg, "rank0_PARA_layer3.swp"))
    y = torch.empty_like(x)
    h = sw.swap_in(did, y, async_op=True)
    assert not sw.is_empty() or h.is_completed()
    sw.synchronize()
    assert torch.equal(x, y) and sw.is_empty()
    grp = NVMeGroup([4096, 2048], sw)
    a, b = torch.randn(4096), torch.randn(2048)
    oid = FlexTrainDataID(FlexTrainDataType.OPTS, 0)
    grp.group_offload(oid, [a, b])
    assert os.path.exists(os.path.join(swap_cfg, "rank0_OPTS_layer0.swp.1"))
    a2, b2 = torch.empty_like(a), torch.empty_like(b)
    grp.group_reload(oid, [a2, b2])
    assert torch.equal(a, a2) and torch.equal(b, b2)
    with pytest.raises(ValueError):
        grp.single_offload(oid, torch.randn(5), 0)
    sw.remove(did)
    assert not os.path.exists(os.path.join(swap_cfg, "rank0_PARA_layer3.swp"))


def test_registered_buffers_become_fixed_requests(tmp_path):
    """io_uring only: transfers that lie inside a registered staging buffer are
    issued as fixed-buffer requests; others stay ordinary; data round-trips in
    both cases; re-registering and dropping the set works while idle."""
    import torch
    from flextrain_b200.memory.nvme_swapper import NVMeEngine
    eng = NVMeEngine(block_size=1 << 16, queue_depth=4, threads=2, engine="auto")
    if eng.kind != "io_uring":
        eng.close()
        pytest.skip("io_uring is not available here")
    staged = torch.arange(1 << 18, dtype=torch.int32)            # 1 MiB
    other = torch.arange(1 << 16, dtype=torch.int32) * 3
    holders = eng.register_buffers([staged])
    path_a, path_b = str(tmp_path / "a.swp"), str(tmp_path / "b.swp")
    eng.write(path_a, staged)
    eng.write(path_b, other)
    fixed_after_writes = eng.stats()["fixed_buffer_requests"]
    if holders:                                                  # the kernel may refuse (memlock limit)
        assert fixed_after_writes == (staged.numel() * 4) // (1 << 16)
    else:
        assert fixed_after_writes == 0
    back = torch.zeros_like(staged)
    eng.read(path_a, back)                                       # not registered: ordinary requests
    assert torch.equal(back, staged)
    assert eng.stats()["fixed_buffer_requests"] == fixed_after_writes
    # a view inside the registered buffer is covered as well
    staged.zero_()
    eng.read(path_a, staged[: 1 << 17])
    assert torch.equal(staged[: 1 << 17], back[: 1 << 17])
    if holders:
        assert eng.stats()["fixed_buffer_requests"] > fixed_after_writes
    assert eng.register_buffers([staged, other]) in (0, 2)       # replace the set
    assert eng.register_buffers([]) == 0                         # drop it
    check = torch.zeros_like(other)
    eng.read(path_b, check)
    assert torch.equal(check, other)
    eng.close()
