"""Every module path of the reference package exists here (scripts written against the
reference import sub-modules directly), and the I/O handle answers to the reference's
method names."""
import importlib

import pytest
import torch

# the reference's package layout (flextrain/**/*.py) minus its unrelated toy script
REFERENCE_MODULES = """
auto_config checkpointing config defaults engine git_version_info_installed llm_func loss_scaler
memory memory.coordinator memory.coordinator.interlayer memory.coordinator.optimizer
memory.coordinator.parameter memory.initializer memory.nvme_swapper memory.pin_memory ops ops.adam
ops.adam.cpu_adam ops.aio ops.op_builder ops.op_builder.async_io ops.op_builder.builder
ops.op_builder.cpu_adam optimizer param_group scheduler utils utils.distributed utils.logging utils.torch
""".split()


@pytest.mark.parametrize("name", REFERENCE_MODULES)
def test_module_exists(name):
    importlib.import_module("flextrain_b200." + name)


def test_version_record_and_torch_helpers():
    from flextrain_b200 import git_version_info_installed as info
    from flextrain_b200.utils import torch as shims
    assert info.version.startswith("0.") and set(info.torch_info) >= {"version", "cuda_version", "nccl_version"}
    assert shims.torch_version_ge("2.0") and not shims.torch_version_ge("99.0")
    assert shims.torch_version_eq(f"{shims.TORCH_MAJOR}.{shims.TORCH_MINOR}")
    assert shims.get_all_gather_function() is torch.distributed.all_gather_into_tensor
    assert shims.get_reduce_scatter_function() is torch.distributed.reduce_scatter_tensor


def test_aio_handle_speaks_the_reference_dialect(tmp_path):
    from flextrain_b200.ops.aio import AsyncIOBuilder, aio_handle, aio_read, aio_write, deepspeed_memcpy
    from flextrain_b200.ops.op_builder.async_io import AsyncIOBuilder as same
    assert AsyncIOBuilder is same
    h = aio_handle(block_size=1 << 16, queue_depth=4, single_submit=False, overlap_events=True,
                   intra_op_parallelism=2)
    assert (h.get_block_size(), h.get_queue_depth(), h.get_intra_op_parallelism()) == (1 << 16, 4, 2)
    assert h.get_overlap_events() and not h.get_single_submit() and h.get_alignment() == 512
    x = h.new_cpu_locked_tensor(1 << 16, torch.empty(0, dtype=torch.float32))
    x.copy_(torch.randn(1 << 16))
    a, b = str(tmp_path / "a.swp"), str(tmp_path / "b.swp")
    assert h.sync_pwrite(x, a) == 0
    assert h.async_pwrite(x, b) == 0 and h.wait() == 1
    y, z = torch.empty_like(x), torch.empty_like(x)
    assert h.async_pread(y, a) == 0 and h.async_pread(z, b) == 0 and h.wait() == 2
    assert torch.equal(x, y) and torch.equal(x, z)
    y.zero_()
    assert h.pread(y, a, True, False) == 0 and torch.equal(x, y)          # validate=True, blocking
    half = x.numel() * 2                                                  # byte offset of the second half
    tail = torch.empty(x.numel() // 2)
    h.read(tail, a, False, half)
    assert torch.equal(tail, x[x.numel() // 2:])
    h.free_cpu_locked_tensor(x)
    h.close()
    # one-shot calls and the host copy
    src = torch.randn(5000)
    c = str(tmp_path / "c.swp")
    assert aio_write(src, c, 1 << 16, 4, False, True, True) == 0
    dst = torch.empty_like(src)
    assert aio_read(dst, c, 1 << 16, 4, False, True, False) == 0 and torch.equal(src, dst)
    dst.zero_()
    assert deepspeed_memcpy(dst, src) == 0 and torch.equal(src, dst)
