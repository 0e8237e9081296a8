"""NVMe tier: swap flat pinned tensors to and from files through the native
asynchronous I/O engine.

Parity: flextrain/memory/nvme_swapper.py:1-245 (``AsyncNVMeSwapper`` :47-158,
``NVMeGroup`` :174-245).  File names are ``<swap_dir>/<FlexTrainDataID>`` and,
for groups, ``<id>.<index>``; the swap directory is emptied when the swapper is
first used.  One engine serves reads and writes (its workers multiplex both),
errors surface as Python exceptions and descriptors are cached and closed with
the engine.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_int, c_int64, c_void_p
from typing import List, Optional, Sequence

import torch

from ..config import get_flextrain_config
from ..utils import distributed as dist
from ..utils.logging import rank0_logger
from . import FlexTrainDataID, Waitable

_ENGINE_CODES = {"auto": 0, "io_uring": 1, "aio": 2, "psync": 3}
_ENGINE_NAMES = {1: "io_uring", 2: "aio", 3: "psync"}


def _lib():
    from ..ops.native import host_lib
    lib = host_lib()
    if not getattr(lib, "_nvme_declared", False):
        lib.ft_nvme_create.restype = c_void_p
        lib.ft_nvme_create.argtypes = [c_int64, c_int, c_int, c_int, c_int]
        lib.ft_nvme_engine_kind.argtypes = [c_void_p]
        lib.ft_nvme_destroy.argtypes = [c_void_p]
        lib.ft_nvme_submit.restype = c_int64
        lib.ft_nvme_submit.argtypes = [c_void_p, c_char_p, c_void_p, c_int64, c_int64, c_int]
        lib.ft_nvme_wait_op.argtypes = [c_void_p, c_int64]
        lib.ft_nvme_wait.restype = c_int64
        lib.ft_nvme_wait.argtypes = [c_void_p]
        lib.ft_nvme_pending.argtypes = [c_void_p]
        lib.ft_nvme_sync_rw.argtypes = [c_void_p, c_char_p, c_void_p, c_int64, c_int64, c_int]
        lib.ft_nvme_forget.argtypes = [c_void_p, c_char_p]
        lib.ft_nvme_open_fds.argtypes = [c_void_p]
        lib.ft_nvme_inject_fault.argtypes = [c_void_p, c_int, c_int]
        lib.ft_nvme_stats.argtypes = [c_void_p, ctypes.POINTER(c_int64), ctypes.POINTER(c_int64)]
        lib.ft_nvme_register_buffers.argtypes = [c_void_p, c_void_p, c_void_p, c_int]
        lib.ft_nvme_fixed_ops.restype = c_int64
        lib.ft_nvme_fixed_ops.argtypes = [c_void_p]
        lib._nvme_declared = True
    return lib


class NVMeError(OSError):
    pass


class AsyncIOHandle(Waitable):
    """Completion of a set of queued transfers."""

    def __init__(self, engine: "NVMeEngine", op_ids: Sequence[int], keep=()):
        self._engine, self._ids, self._keep = engine, list(op_ids), keep

    def wait(self):
        ids, self._ids = self._ids, []
        first = 0
        for i in ids:
            rc = self._engine._wait_op(i)
            if rc and not first:
                first = rc
        self._keep = ()
        if first:
            raise NVMeError(-first, f"NVMe transfer failed: {os.strerror(-first)}")

    def is_completed(self):
        return not self._ids


class NVMeEngine:
    """Thin object wrapper over the native engine (``ft_nvme_*``)."""

    def __init__(self, block_size=1 << 20, queue_depth=8, threads=4, engine="auto", o_direct=True):
        self._lib = _lib()
        self._h = self._lib.ft_nvme_create(block_size, queue_depth, threads,
                                           _ENGINE_CODES[engine], int(o_direct))
        if not self._h:
            raise NVMeError("could not create the NVMe engine")
        self.kind = _ENGINE_NAMES.get(self._lib.ft_nvme_engine_kind(self._h), "?")

    def close(self):
        if self._h:
            self._lib.ft_nvme_destroy(self._h)
            self._h = None

    __del__ = close

    def submit(self, path: str, tensor: torch.Tensor, write: bool, file_offset: int = 0) -> int:
        if tensor.device.type != "cpu" or not tensor.is_contiguous():
            raise ValueError("NVMe transfers need contiguous CPU tensors")
        rc = self._lib.ft_nvme_submit(self._h, path.encode(), tensor.data_ptr(),
                                      tensor.numel() * tensor.element_size(), file_offset, int(write))
        if rc < 0:
            raise NVMeError(-rc, f"cannot queue NVMe transfer on {path}: {os.strerror(-rc)}")
        return rc

    def _wait_op(self, op_id: int) -> int:
        return self._lib.ft_nvme_wait_op(self._h, op_id)

    def wait_all(self) -> int:
        rc = self._lib.ft_nvme_wait(self._h)
        if rc < 0:
            raise NVMeError(-rc, f"NVMe transfer failed: {os.strerror(-rc)}")
        return rc

    def pending(self) -> int:
        return self._lib.ft_nvme_pending(self._h)

    def read(self, path, tensor, file_offset=0):
        rc = self._lib.ft_nvme_sync_rw(self._h, path.encode(), tensor.data_ptr(),
                                       tensor.numel() * tensor.element_size(), file_offset, 0)
        if rc:
            raise NVMeError(-rc, f"NVMe read of {path} failed: {os.strerror(-rc)}")

    def write(self, path, tensor, file_offset=0):
        rc = self._lib.ft_nvme_sync_rw(self._h, path.encode(), tensor.data_ptr(),
                                       tensor.numel() * tensor.element_size(), file_offset, 1)
        if rc:
            raise NVMeError(-rc, f"NVMe write of {path} failed: {os.strerror(-rc)}")

    def forget(self, path):
        return self._lib.ft_nvme_forget(self._h, path.encode())

    def open_fds(self) -> int:
        return self._lib.ft_nvme_open_fds(self._h)

    def inject_fault(self, kind: str, count: int = 1):
        self._lib.ft_nvme_inject_fault(self._h, {"eio": 1, "short": 2}[kind], count)

    def stats(self):
        r, w = c_int64(0), c_int64(0)
        self._lib.ft_nvme_stats(self._h, ctypes.byref(r), ctypes.byref(w))
        return {"bytes_read": r.value, "bytes_written": w.value,
                "fixed_buffer_requests": int(self._lib.ft_nvme_fixed_ops(self._h))}

    def register_buffers(self, tensors: Sequence[torch.Tensor]) -> int:
        """Register the storage of ``tensors`` (contiguous CPU staging buffers)
        with the io_uring workers; transfers inside them then run as
        fixed-buffer requests.  Replaces any earlier set.  Returns how many
        workers hold the registration (0: not io_uring, or the kernel refused -
        transfers stay ordinary requests).  No transfer may be pending."""
        tensors = [t for t in tensors if t.numel() > 0]
        n = len(tensors)
        ptrs = (c_void_p * max(n, 1))(*[t.data_ptr() for t in tensors])
        lens = (c_int64 * max(n, 1))(*[t.numel() * t.element_size() for t in tensors])
        rc = self._lib.ft_nvme_register_buffers(self._h, ptrs, lens, n)
        if rc < 0:
            raise NVMeError(-rc, f"cannot register NVMe staging buffers: {os.strerror(-rc)}")
        return rc


class AsyncNVMeSwapper:
    def __init__(self, swap_dir: Optional[str] = None, engine: Optional[NVMeEngine] = None):
        self._cfg = get_flextrain_config().nvme_swap
        self.swap_dir = swap_dir or self._cfg.swap_dir
        self._engine = engine
        self._inflight: List[AsyncIOHandle] = []
        self._ready = False
        self._staging: List[torch.Tensor] = []      # pinned buffers every transfer goes through
        self._staging_dirty = False

    def _init(self):
        if self._ready:
            return
        self._ready = True
        if self._engine is None:
            c = self._cfg
            self._engine = NVMeEngine(c.aio_block_size, c.aio_queue_depth, c.aio_thread_count,
                                      c.io_engine)
        # every rank wipes only its own files so concurrent ranks do not race
        os.makedirs(self.swap_dir, exist_ok=True)
        prefix = f"rank{dist.get_rank()}_"
        for name in os.listdir(self.swap_dir):
            if name.startswith(prefix) and ".swp" in name:
                os.remove(os.path.join(self.swap_dir, name))
        rank0_logger.info(f"NVMe swapper ready: dir={self.swap_dir} engine={self._engine.kind}")

    @property
    def engine(self) -> NVMeEngine:
        self._init()
        return self._engine

    def _filename(self, data_id) -> str:
        return os.path.join(self.swap_dir, str(data_id))

    def register_staging(self, tensor: torch.Tensor):
        """Tell the swapper that ``tensor`` is a long-lived staging buffer of the
        NVMe tier.  The set is registered with the engine (io_uring fixed
        buffers) at the next moment no transfer is pending."""
        if tensor is not None and tensor.numel() > 0 and tensor.device.type == "cpu":
            self._staging.append(tensor)
            self._staging_dirty = True

    def _register_if_idle(self):
        if self._staging_dirty and self._engine.pending() == 0:
            self._staging_dirty = False
            try:
                self._engine.register_buffers(self._staging)
            except NVMeError as exc:                 # registration is an optimisation only
                if exc.errno == 16:                  # EBUSY: a transfer started meanwhile, try later
                    self._staging_dirty = True
                else:
                    rank0_logger.warning(f"NVMe staging buffers not registered: {exc}")

    def _swap(self, data_ids, tensors, write: bool, async_op: bool):
        self._init()
        self._register_if_idle()
        if isinstance(data_ids, (FlexTrainDataID, str)):
            data_ids, tensors = [data_ids], [tensors]
        ids = []
        for did, t in zip(data_ids, tensors):
            if t.numel() == 0:
                continue
            ids.append(self._engine.submit(self._filename(did), t, write))
        handle = AsyncIOHandle(self._engine, ids, keep=tuple(tensors))
        if async_op:
            self._inflight.append(handle)
            return handle
        handle.wait()
        return handle

    @staticmethod
    def _count(kind, tensors):
        from . import TRAFFIC
        ts = [tensors] if isinstance(tensors, torch.Tensor) else list(tensors)
        TRAFFIC.add(kind, sum(t.numel() * t.element_size() for t in ts))

    def swap_out(self, data_ids, tensors, async_op: bool = False):
        self._count("nvme_write", tensors)
        return self._swap(data_ids, tensors, True, async_op)

    def swap_in(self, data_ids, tensors, async_op: bool = False):
        self._count("nvme_read", tensors)
        return self._swap(data_ids, tensors, False, async_op)

    def synchronize(self):
        handles, self._inflight = self._inflight, []
        first = None
        for h in handles:
            try:
                h.wait()
            except NVMeError as e:
                first = first or e
        if first:
            raise first

    def is_empty(self) -> bool:
        self._inflight = [h for h in self._inflight if not h.is_completed()]
        return not self._inflight

    def remove(self, data_id):
        path = self._filename(data_id)
        if self._ready:
            self._engine.forget(path)
        if os.path.exists(path):
            os.remove(path)


class NVMeGroup:
    """A fixed tuple of sub-files ``<id>.<index>`` with per-member sizes."""

    def __init__(self, numels: Sequence[int], swapper: Optional[AsyncNVMeSwapper] = None):
        self._numels = tuple(int(n) for n in numels)
        self._swapper = swapper

    @property
    def swapper(self) -> AsyncNVMeSwapper:
        return self._swapper or get_nvme_swapper()

    @staticmethod
    def _name(prefix, index):
        return f"{prefix}.{index}"

    def _check(self, index, tensor):
        if tensor.numel() != self._numels[index]:
            raise ValueError(f"group member {index} holds {self._numels[index]} elements, "
                             f"got {tensor.numel()}")

    def single_offload(self, prefix, tensor, index, async_op=False):
        self._check(index, tensor)
        return self.swapper.swap_out(self._name(prefix, index), tensor, async_op)

    def single_reload(self, prefix, tensor, index, async_op=False):
        self._check(index, tensor)
        return self.swapper.swap_in(self._name(prefix, index), tensor, async_op)

    def group_offload(self, prefix, tensors, async_op=False):
        for i, t in enumerate(tensors):
            self._check(i, t)
        return self.swapper.swap_out([self._name(prefix, i) for i in range(len(tensors))],
                                     list(tensors), async_op)

    def group_reload(self, prefix, tensors, async_op=False):
        for i, t in enumerate(tensors):
            self._check(i, t)
        return self.swapper.swap_in([self._name(prefix, i) for i in range(len(tensors))],
                                    list(tensors), async_op)


_SWAPPER: Optional[AsyncNVMeSwapper] = None


def get_nvme_swapper() -> AsyncNVMeSwapper:
    global _SWAPPER
    if _SWAPPER is None:
        _SWAPPER = AsyncNVMeSwapper()
    return _SWAPPER


def reset_nvme_swapper():
    global _SWAPPER
    if _SWAPPER is not None and _SWAPPER._engine is not None:
        _SWAPPER._engine.close()
    _SWAPPER = None


def swap_in_tensors(swap_handle, tensor_buffers, swap_paths):
    """Queue one asynchronous read per (buffer, path) pair on an ``aio_handle``-like object
    (flextrain/memory/nvme_swapper.py:12-14); the caller ``wait()``s on the handle."""
    for buffer, path in zip(tensor_buffers, swap_paths):
        if swap_handle.async_pread(buffer, path, 0) != 0:
            raise NVMeError(f"cannot queue the read of {path}")


def swap_out_tensors(swap_handle, tensor_buffers, swap_paths):
    """Queue one asynchronous write per (buffer, path) pair (flextrain/memory/nvme_swapper.py:17-19)."""
    for buffer, path in zip(tensor_buffers, swap_paths):
        if swap_handle.async_pwrite(buffer, path, 0) != 0:
            raise NVMeError(f"cannot queue the write of {path}")
