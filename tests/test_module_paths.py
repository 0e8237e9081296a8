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


def test_helper_names_of_the_reference_modules():
    import numpy as np
    from flextrain_b200 import memory as M
    from flextrain_b200.loss_scaler import INITIAL_LOSS_SCALE, MIN_LOSS_SCALE, DynamicLossScaler, to_python_float
    from flextrain_b200.memory.coordinator.interlayer import InterLayerTask
    from flextrain_b200.memory.nvme_swapper import AsyncIOHandle
    from flextrain_b200.param_group import flatten_list, is_same_param_group, reshape_list
    from flextrain_b200.utils.distributed import is_single_process
    grid = reshape_list([torch.zeros(2), torch.ones(2), torch.zeros(3), torch.ones(3)], [2, 2])
    assert isinstance(grid, np.ndarray) and grid.shape == (2, 2) and grid[1, 0].numel() == 3
    assert flatten_list([1, [2, [3, 4]], 5]) == [1, 2, 3, 4, 5] and flatten_list(7) == [7]
    g = {"lr": 1.0}
    assert is_same_param_group(g, g) and not is_same_param_group(g, dict(g))
    assert to_python_float(torch.tensor([2.5])) == 2.5 and to_python_float(3) == 3.0
    scaler = DynamicLossScaler(**{INITIAL_LOSS_SCALE: 2.0 ** 8, MIN_LOSS_SCALE: 1.0})
    assert scaler.loss_scale == 256.0
    assert M.get_page_aligned_numel(5, 4) == 1024 and M.get_partition_aligned_numel(5, 3, 2) == 6144
    before = M.get_allocated_dram_size()
    M.allocate_memory(100, torch.float32, "cpu", pinned=False)
    assert M.get_allocated_dram_size() - before == 400 and M.get_allocated_vram_size() >= 0
    assert M.AsyncIOHandle is AsyncIOHandle and M.FlexTrainDataStream is not None
    task = InterLayerTask(True, 2, 1, torch.ones(1))
    assert (task.unit, task.micro_batch) == (2, 1) and task.tensor.item() == 1.0
    assert isinstance(is_single_process(), bool)


def test_swap_helpers_on_an_aio_handle(tmp_path):
    from flextrain_b200.memory.nvme_swapper import swap_in_tensors, swap_out_tensors
    from flextrain_b200.ops.aio import aio_handle
    h = aio_handle(intra_op_parallelism=2)
    xs = [torch.randn(4096), torch.randn(8192)]
    paths = [str(tmp_path / "x0.swp"), str(tmp_path / "x1.swp")]
    swap_out_tensors(h, xs, paths)
    assert h.wait() == 2
    ys = [torch.empty_like(x) for x in xs]
    swap_in_tensors(h, ys, paths)
    assert h.wait() == 2 and all(torch.equal(a, b) for a, b in zip(xs, ys))
    h.close()


def test_builder_version_helpers():
    from flextrain_b200.ops.op_builder import CPUAdamBuilder
    from flextrain_b200.ops.op_builder import builder as B
    assert issubclass(CPUAdamBuilder, B.CPUOpBuilder)
    assert B.get_default_compute_capabilities() == "10.0a"
    if B.nvcc_path():
        major, minor = B.installed_cuda_version()
        assert (major, minor) >= (12, 8) and B.assert_no_cuda_mismatch("test")
    else:
        with pytest.raises(B.MissingCUDAException):
            B.installed_cuda_version()
