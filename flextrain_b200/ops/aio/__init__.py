"""Asynchronous file I/O with the call surface of the reference's ``aio`` extension.

Parity: the pybind module of flextrain/ops/csrc/aio/py_lib/py_ds_aio.cpp:14-127
(``aio_read``, ``aio_write``, ``deepspeed_memcpy`` and the ``aio_handle`` class with
``read / write / pread / pwrite / sync_pread / sync_pwrite / async_pread / async_pwrite /
wait``, the getters and the locked-tensor pair), loaded in the reference through
flextrain/ops/aio/__init__.py.  Here the same names sit on the io_uring engine of
``csrc/host/nvme_engine.cpp`` (``memory/nvme_swapper.NVMeEngine``); there is nothing to
JIT-compile, so ``AsyncIOBuilder().load()`` returns this module.

Differences kept on purpose: failures raise ``NVMeError`` instead of tripping a C
``assert``; file descriptors are cached per path and closed with the handle; ``validate``
re-reads through the page cache like the reference and raises on a mismatch.
"""
from __future__ import annotations

import os
from typing import Union

import torch

from ...memory.nvme_swapper import NVMeEngine, NVMeError
from ...memory.pin_memory import free_cpu_locked_tensor, host_memcpy, new_cpu_locked_tensor
from ..op_builder import AsyncIOBuilder

__all__ = ["aio_handle", "aio_read", "aio_write", "deepspeed_memcpy", "AsyncIOBuilder", "NVMeError"]

_ALIGNMENT = 512          # O_DIRECT: offsets and lengths in units of the logical block size


def _validate(buffer: torch.Tensor, filename: str, file_offset: int):
    nbytes = buffer.numel() * buffer.element_size()
    with open(filename, "rb") as f:
        f.seek(file_offset)
        data = f.read(nbytes)
    mine = buffer.contiguous().view(torch.uint8).numpy().tobytes()
    if data != mine:
        raise NVMeError(f"validation of {filename} failed: file and buffer differ")


def _path_of(target: Union[str, int]) -> str:
    """The reference also accepts an open file descriptor; its path is looked up."""
    if isinstance(target, int):
        return os.readlink(f"/proc/self/fd/{target}")
    return os.fspath(target)


class aio_handle:                                            # noqa: N801 (the reference's class name)
    def __init__(self, block_size: int = 1024 * 1024, queue_depth: int = 128, single_submit: bool = False,
                 overlap_events: bool = False, intra_op_parallelism: int = 1):
        self._block_size, self._queue_depth = int(block_size), int(queue_depth)
        self._single_submit, self._overlap_events = bool(single_submit), bool(overlap_events)
        self._threads = max(1, int(intra_op_parallelism))
        self._engine = NVMeEngine(block_size=self._block_size, queue_depth=self._queue_depth,
                                  threads=self._threads)
        self._inflight = 0

    # ------------------------------------------------------------------ getters
    def get_block_size(self): return self._block_size
    def get_queue_depth(self): return self._queue_depth
    def get_single_submit(self): return self._single_submit
    def get_overlap_events(self): return self._overlap_events
    def get_intra_op_parallelism(self): return self._threads
    def get_alignment(self): return _ALIGNMENT

    # ---------------------------------------------------------------- transfers
    def read(self, buffer, filename, validate=False, file_offset=0):
        self._engine.read(_path_of(filename), buffer, file_offset)
        if validate:
            _validate(buffer, _path_of(filename), file_offset)
        return 0

    def write(self, buffer, filename, validate=False, file_offset=0):
        self._engine.write(_path_of(filename), buffer, file_offset)
        if validate:
            _validate(buffer, _path_of(filename), file_offset)
        return 0

    def pread(self, buffer, filename, validate=False, async_op=False, file_offset=0, **kw):
        async_op = kw.get("async", async_op)                 # the reference's keyword is ``async``
        if not async_op:
            return self.read(buffer, filename, validate, file_offset)
        self._engine.submit(_path_of(filename), buffer, False, file_offset)
        self._inflight += 1
        return 0

    def pwrite(self, buffer, filename, validate=False, async_op=False, file_offset=0, **kw):
        async_op = kw.get("async", async_op)
        if not async_op:
            return self.write(buffer, filename, validate, file_offset)
        self._engine.submit(_path_of(filename), buffer, True, file_offset)
        self._inflight += 1
        return 0

    def sync_pread(self, buffer, filename, file_offset=0):
        return self.pread(buffer, filename, False, False, file_offset)

    def sync_pwrite(self, buffer, filename, file_offset=0):
        return self.pwrite(buffer, filename, False, False, file_offset)

    def async_pread(self, buffer, filename, file_offset=0):
        return self.pread(buffer, filename, False, True, file_offset)

    def async_pwrite(self, buffer, filename, file_offset=0):
        return self.pwrite(buffer, filename, False, True, file_offset)

    def wait(self) -> int:
        """Waits for every asynchronous transfer; returns how many completed."""
        self._engine.wait_all()
        done, self._inflight = self._inflight, 0
        return done

    # ------------------------------------------------------------ locked tensors
    def new_cpu_locked_tensor(self, num_elem: int, example_tensor: torch.Tensor) -> torch.Tensor:
        return new_cpu_locked_tensor(int(num_elem), example_tensor.dtype)

    def free_cpu_locked_tensor(self, tensor: torch.Tensor):
        return free_cpu_locked_tensor(tensor)

    def close(self):
        self._engine.close()


def _one_shot(buffer, filename, block_size, queue_depth, write, validate):
    h = aio_handle(block_size, queue_depth)
    try:
        (h.write if write else h.read)(buffer, filename, validate)
    finally:
        h.close()
    return 0


def aio_read(buffer, filename, block_size=1 << 20, queue_depth=8, single_submit=False, overlap_events=True,
             validate=False):
    """Blocking one-off read of the whole buffer (flextrain/ops/csrc/aio/py_lib/deepspeed_py_aio.cpp:81-123)."""
    return _one_shot(buffer, filename, block_size, queue_depth, False, validate)


def aio_write(buffer, filename, block_size=1 << 20, queue_depth=8, single_submit=False, overlap_events=True,
              validate=False):
    """Blocking one-off write (flextrain/ops/csrc/aio/py_lib/deepspeed_py_aio.cpp:39-79)."""
    return _one_shot(buffer, filename, block_size, queue_depth, True, validate)


def deepspeed_memcpy(dest: torch.Tensor, src: torch.Tensor):
    """Multi-threaded streaming host copy (flextrain/ops/csrc/aio/py_lib/deepspeed_py_copy.cpp:25-135)."""
    host_memcpy(dest, src)
    return 0
