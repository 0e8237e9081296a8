"""One process per GPU on a single node; thin wrappers over torch.distributed.

Parity: flextrain/utils/distributed.py:1-199 and flextrain/utils/torch.py:1-63.
Every wrapper degenerates to a finished handle when the world size is 1, so a
single-GPU run needs no process group.  Two backends are served:

* ``nccl``  - the B200 path (device = ``cuda:LOCAL_RANK``);
* ``gloo``  - CPU ranks for tests; gloo has neither reduce-scatter nor AVG, so
  those are emulated with an all-reduce (SUM) and a local slice / divide.
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as tdist
from torch.distributed import ReduceOp

from ..defaults import (PROCESS_GROUP_TIMEOUT_DEFAULT, TORCH_DISTRIBUTED_BACKEND_DEFAULT,
                        TORCH_DISTRIBUTED_INIT_METHOD_DEFAULT)
from .logging import rank0_logger

_INITIALIZED = False
_RANK = 0
_WORLD_SIZE = 1
_BACKEND: Optional[str] = None
_DEVICE: Optional[torch.device] = None


class DummyHandle:
    """A finished piece of asynchronous work."""

    def wait(self):
        return None

    def is_completed(self):
        return True


def init_distributed(dist_backend=TORCH_DISTRIBUTED_BACKEND_DEFAULT,
                     timeout=PROCESS_GROUP_TIMEOUT_DEFAULT,
                     init_method=TORCH_DISTRIBUTED_INIT_METHOD_DEFAULT,
                     force_init=True, rank=-1, world_size=-1):
    """Create the default process group (unless one exists) and bind this
    process to its device.  With ``force_init=False`` a WORLD_SIZE of 1 skips the
    process group altogether.  CPU threads are budgeted as
    ``cpu_count // WORLD_SIZE`` per rank: that is the host Adam's share."""
    global _INITIALIZED, _RANK, _WORLD_SIZE, _BACKEND, _DEVICE
    if _INITIALIZED:
        return
    _INITIALIZED = True

    env_world = int(os.getenv("WORLD_SIZE", "0"))
    if world_size > 0:
        env_world = world_size
    if env_world == 0:
        rank0_logger.info("WORLD_SIZE is not set: running as a single process")
        env_world = 1
    os.environ.setdefault("WORLD_SIZE", str(env_world))

    if dist_backend == "nccl" and not torch.cuda.is_available():
        rank0_logger.warning("CUDA is not available: falling back to the gloo backend on CPU")
        dist_backend = "gloo"
    _BACKEND = dist_backend

    if env_world == 1 and not force_init and not tdist.is_initialized():
        _RANK, _WORLD_SIZE = 0, 1
        _bind_device(int(os.getenv("LOCAL_RANK", "0")))
        return

    threads = max(1, (os.cpu_count() or 1) // env_world)
    if env_world > 1:
        if int(os.getenv("OMP_NUM_THREADS", "0")) <= threads:
            os.environ["OMP_NUM_THREADS"] = str(threads)
        if torch.get_num_threads() != threads:
            torch.set_num_threads(threads)

    if not tdist.is_initialized():
        kwargs = dict(backend=dist_backend, timeout=timeout, init_method=init_method)
        if rank >= 0:
            kwargs["rank"] = rank
        if world_size > 0:
            kwargs["world_size"] = world_size
        if dist_backend == "nccl":
            local = int(os.getenv("LOCAL_RANK", os.getenv("RANK", "0") if rank < 0 else rank))
            torch.cuda.set_device(local)
            kwargs["device_id"] = torch.device("cuda", local)
        tdist.init_process_group(**kwargs)
    else:
        _BACKEND = tdist.get_backend()

    _RANK = tdist.get_rank()
    _WORLD_SIZE = tdist.get_world_size()
    # single node: the local rank is the global rank
    _bind_device(int(os.getenv("LOCAL_RANK", str(_RANK))))
    rank0_logger.info(f"distributed ready: backend={_BACKEND} world={_WORLD_SIZE} "
                      f"device={_DEVICE} host-threads/rank={threads}")


def _bind_device(local_rank: int):
    global _DEVICE
    if _BACKEND != "gloo" and torch.cuda.is_available():
        torch.cuda.set_device(local_rank)
        _DEVICE = torch.device("cuda", local_rank)
        if os.getenv("FLEXTRAIN_NUMA", "0") == "1":
            # threads started from here on (host Adam, NVMe workers, the update worker) and the
            # pages they touch first stay on the socket of this rank's GPU
            from .numa import bind_to_gpu_node
            bind_to_gpu_node(local_rank, int(os.getenv("LOCAL_WORLD_SIZE", os.getenv("WORLD_SIZE", "1"))))
    else:
        _DEVICE = torch.device("cpu")


def _ensure():
    if not _INITIALIZED:
        init_distributed(force_init=False)


def is_single_process() -> bool:
    """True when this run has one rank (flextrain/utils/distributed.py:134-136)."""
    _ensure()
    return _WORLD_SIZE == 1


def shutdown():
    """Destroy the process group and forget all state (tests)."""
    global _INITIALIZED, _RANK, _WORLD_SIZE, _BACKEND, _DEVICE
    if tdist.is_initialized():
        tdist.destroy_process_group()
    _INITIALIZED, _RANK, _WORLD_SIZE, _BACKEND, _DEVICE = False, 0, 1, None, None


def is_initialized() -> bool:
    return _INITIALIZED


def get_rank() -> int:
    _ensure()
    return _RANK


def get_world_size() -> int:
    _ensure()
    return _WORLD_SIZE


def get_backend() -> Optional[str]:
    _ensure()
    return _BACKEND


def current_device() -> torch.device:
    """The device this rank computes on: ``cuda:LOCAL_RANK`` or ``cpu``."""
    _ensure()
    return _DEVICE


def is_cuda() -> bool:
    return current_device().type == "cuda"


def _native_avg() -> bool:
    return _BACKEND == "nccl"


def barrier(group=None):
    _ensure()
    if _WORLD_SIZE > 1:
        tdist.barrier(group=group)


def print_rank0(*args, **kwargs):
    if get_rank() == 0:
        print(*args, **kwargs, flush=True)


def print_rank_by_rank(*args, **kwargs):
    for r in range(get_world_size()):
        if r == get_rank():
            print(f"[rank {r}]", *args, **kwargs, flush=True)
        barrier()


# The collectives below take their arguments in the order of the reference's wrappers
# (flextrain/utils/distributed.py:171-199): ``group`` before ``async_op``.  The engine only
# ever uses the default group; a caller's own group is passed through to torch.distributed.
def broadcast(tensor: torch.Tensor, src: int = 0, group=None, async_op: bool = False):
    _ensure()
    if _WORLD_SIZE == 1:
        return DummyHandle()
    return tdist.broadcast(tensor, src, group=group, async_op=async_op) or DummyHandle()


def all_gather(output: torch.Tensor, shard: torch.Tensor, group=None, async_op: bool = False):
    """``output`` (W * n elements) receives every rank's ``shard`` (n) in rank order."""
    _ensure()
    if _WORLD_SIZE == 1:
        if output.data_ptr() != shard.data_ptr():
            output.view(-1)[: shard.numel()].copy_(shard.view(-1), non_blocking=True)
        return DummyHandle()
    return tdist.all_gather_into_tensor(output, shard, group=group, async_op=async_op) or DummyHandle()


class _PostOp:
    """Finishes an emulated collective (divide / slice) after the real one."""

    def __init__(self, work, fn):
        self._work, self._fn = work, fn

    def wait(self):
        if self._work is not None:
            self._work.wait()
            self._work = None
        if self._fn is not None:
            self._fn()
            self._fn = None

    def is_completed(self):
        return self._work is None and self._fn is None


def all_reduce(tensor: torch.Tensor, op=ReduceOp.SUM, group=None, async_op: bool = False):
    _ensure()
    if _WORLD_SIZE == 1:
        return DummyHandle()
    if op == ReduceOp.AVG and not _native_avg():
        work = tdist.all_reduce(tensor, ReduceOp.SUM, group=group, async_op=async_op)
        post = _PostOp(work if async_op else None, lambda: tensor.div_(tdist.get_world_size(group)))
        if not async_op:
            post.wait()
            return DummyHandle()
        return post
    return tdist.all_reduce(tensor, op, group=group, async_op=async_op) or DummyHandle()


def reduce_scatter(output: torch.Tensor, full: torch.Tensor, op=ReduceOp.SUM, group=None,
                   async_op: bool = False):
    """``output`` (n) receives this rank's slice of the reduction of ``full`` (W * n).
    ``output`` may alias ``full``'s own slice (the reference reduces in place:
    coordinator/optimizer.py:550-552)."""
    _ensure()
    if _WORLD_SIZE == 1:
        if output.data_ptr() != full.data_ptr():
            output.view(-1).copy_(full.view(-1)[: output.numel()], non_blocking=True)
        return DummyHandle()
    if _BACKEND == "nccl":
        return tdist.reduce_scatter_tensor(output, full, op, group=group, async_op=async_op) or DummyHandle()
    # gloo: all-reduce a scratch copy, keep the local slice
    scratch = full.detach().clone()
    work = tdist.all_reduce(scratch, ReduceOp.SUM, group=group, async_op=async_op)
    n = output.numel()
    g_rank, g_world = tdist.get_rank(group), tdist.get_world_size(group)

    def finish():
        piece = scratch.view(-1)[g_rank * n:(g_rank + 1) * n]
        if op == ReduceOp.AVG:
            piece = piece / g_world
        output.view(-1).copy_(piece)

    post = _PostOp(work if async_op else None, finish)
    if not async_op:
        post.wait()
        return DummyHandle()
    return post


def all_reduce_scalar(value: float, op=ReduceOp.SUM) -> float:
    """World reduction of a Python number (planner statistics, overflow flags)."""
    _ensure()
    if _WORLD_SIZE == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64 if _BACKEND == "gloo" else torch.float32,
                     device=current_device())
    all_reduce(t, op)
    return float(t.item())
