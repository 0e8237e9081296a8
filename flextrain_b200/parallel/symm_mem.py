"""Symmetric peer memory on one NVSwitch node.

Every rank allocates the same buffer with ``cudaMalloc`` (outside PyTorch's
caching allocator, so the whole allocation can be exported), publishes its CUDA
IPC handle through the process group and maps every peer's buffer.  Kernels then
read and write other GPUs' memory with plain loads and stores.  The reference
has no counterpart: its only transports are NCCL collectives
(flextrain/utils/distributed.py:139-199).
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as tdist

from ..ops.native import cuda_lib
from ..utils import distributed as dist

_DECLARED = False


def _lib():
    global _DECLARED
    lib = cuda_lib()
    if not _DECLARED:
        lib.ft_symm_alloc.restype = ctypes.c_void_p
        lib.ft_symm_alloc.argtypes = [ctypes.c_size_t]
        lib.ft_symm_free.argtypes = [ctypes.c_void_p]
        lib.ft_ipc_get_handle.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        lib.ft_ipc_open.restype = ctypes.c_void_p
        lib.ft_ipc_open.argtypes = [ctypes.c_void_p]
        lib.ft_ipc_close.argtypes = [ctypes.c_void_p]
        lib.ft_can_access_peer.argtypes = [ctypes.c_int, ctypes.c_int]
        _DECLARED = True
    return lib


class _RawCudaMemory:
    """Exposes a raw device allocation through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 3, "strides": None}


def tensor_from_ptr(ptr: int, nbytes: int, dtype: torch.dtype, device) -> torch.Tensor:
    raw = torch.as_tensor(_RawCudaMemory(ptr, nbytes), device=device)
    return raw.view(dtype)


def peer_access_available() -> bool:
    """True when every pair of ranks on this node can address each other."""
    if not dist.is_cuda():
        return False
    world = dist.get_world_size()
    if world == 1:
        return True
    lib = _lib()
    me = torch.cuda.current_device()
    ok = all(lib.ft_can_access_peer(me, r) for r in range(world) if r != me)
    return bool(dist.all_reduce_scalar(1.0 if ok else 0.0, dist.ReduceOp.MIN) > 0.5)


class SymmetricBuffer:
    """``nbytes`` of device memory on every rank, all of them mapped locally.

    ``ptrs[r]`` is this process's address of rank ``r``'s buffer.  Collective:
    every rank must construct its buffers in the same order."""

    def __init__(self, nbytes: int):
        lib = _lib()
        self.nbytes = int(nbytes)
        self.world, self.rank = dist.get_world_size(), dist.get_rank()
        self.device = dist.current_device()
        self._own = lib.ft_symm_alloc(self.nbytes)
        if not self._own:
            raise MemoryError(f"symmetric allocation of {nbytes} bytes failed")
        self.ptrs: List[int] = [0] * self.world
        self.ptrs[self.rank] = self._own
        self._opened: List[int] = []
        if self.world > 1:
            handle = (ctypes.c_uint8 * 64)()
            rc = lib.ft_ipc_get_handle(self._own, handle)
            if rc:
                raise RuntimeError(f"cudaIpcGetMemHandle failed with {rc}")
            mine = torch.tensor(list(bytes(handle)), dtype=torch.uint8, device=self.device)
            every = torch.empty(self.world * 64, dtype=torch.uint8, device=self.device)
            tdist.all_gather_into_tensor(every, mine)
            every = every.cpu()
            for r in range(self.world):
                if r == self.rank:
                    continue
                h = (ctypes.c_uint8 * 64)(*every[r * 64:(r + 1) * 64].tolist())
                p = lib.ft_ipc_open(h)
                if not p:
                    raise RuntimeError(f"cudaIpcOpenMemHandle for rank {r} failed")
                self.ptrs[r] = p
                self._opened.append(p)

    def tensor(self, dtype: torch.dtype, rank: Optional[int] = None) -> torch.Tensor:
        """Flat view of rank ``rank``'s buffer (default: own)."""
        r = self.rank if rank is None else rank
        return tensor_from_ptr(self.ptrs[r], self.nbytes, dtype, self.device)

    def ptr_array(self):
        return (ctypes.c_void_p * self.world)(*self.ptrs)

    def close(self):
        lib = _lib()
        for p in self._opened:
            lib.ft_ipc_close(p)
        self._opened = []
        if self._own:
            if self.world > 1:
                dist.barrier()
            lib.ft_symm_free(self._own)
            self._own = 0


class FlagPage(SymmetricBuffer):
    """4 KiB of 32-bit sequence words per rank: row ``slot``, column ``writer``."""

    ROWS = 128

    def __init__(self):
        super().__init__(self.ROWS * 8 * 4)
        self._seq = {}

    def next_seq(self, site: str) -> int:
        self._seq[site] = self._seq.get(site, 0) + 1
        return self._seq[site]


_FLAG_PAGE: Optional[FlagPage] = None


def get_flag_page() -> FlagPage:
    """The process-wide flag page (collective on first use)."""
    global _FLAG_PAGE
    if _FLAG_PAGE is None:
        _FLAG_PAGE = FlagPage()
    return _FLAG_PAGE


def reset_flag_page():
    global _FLAG_PAGE
    if _FLAG_PAGE is not None:
        _FLAG_PAGE.close()
    _FLAG_PAGE = None
