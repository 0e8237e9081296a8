"""Page-locked host memory: an exact-size native pool and, for callers that
must live with a power-of-two allocator, the waste-minimising block packer.

Parity: flextrain/memory/pin_memory.py:1-171 (``allocate_optimal`` DP :7-73,
``allocate_pin_memory_blocks`` :100-171) and the pinned tensor manager of the
reference's AIO extension (flextrain/ops/csrc/aio/py_lib/deepspeed_pin_tensor.cpp).
The native pool (``ft_pinned_alloc`` in the CUDA library) hands out exact sizes
with ``cudaHostAlloc``, so the packer is only needed when that library is
absent and PyTorch's caching pinned allocator (which rounds every request up to
a power of two) has to be used.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch

from . import allocate_memory


def _next_pow2(n: int) -> int:
    return 1 if n <= 1 else 1 << (n - 1).bit_length()


def allocate_optimal(num_blocks: int, block_bytes: int) -> List[int]:
    """Split ``num_blocks`` equal blocks into groups so that the sum over groups
    of ``next_pow2(group_blocks * block_bytes)`` is minimal.  Returns the group
    sizes (in blocks), largest first.  O(n^2) dynamic programme."""
    if num_blocks <= 0:
        return []
    cost = [0] * (num_blocks + 1)
    take = [0] * (num_blocks + 1)
    for n in range(1, num_blocks + 1):
        best, best_k = None, 0
        for k in range(1, n + 1):
            c = _next_pow2(k * block_bytes) + cost[n - k]
            if best is None or c < best or (c == best and k > best_k):
                best, best_k = c, k
        cost[n], take[n] = best, best_k
    groups, n = [], num_blocks
    while n:
        groups.append(take[n])
        n -= take[n]
    return sorted(groups, reverse=True)


def packing_waste(groups: Sequence[int], block_bytes: int) -> int:
    return sum(_next_pow2(g * block_bytes) - g * block_bytes for g in groups)


def allocate_pin_memory_blocks(numel: int, dtype: torch.dtype, shape: Tuple[int, ...]):
    """``prod(shape)`` pinned flat buffers of ``numel`` elements each, as nested
    lists indexed like ``shape``.  With the native pool one exact allocation is
    carved up; otherwise blocks are packed into power-of-two chunks."""
    total = 1
    for s in shape:
        total *= s
    itemsize = torch.empty((), dtype=dtype).element_size()
    blocks: List[torch.Tensor] = []
    use_native = False
    if torch.cuda.is_available():
        try:
            from ..ops.native import cuda_lib
            cuda_lib()
            use_native = True
        except Exception:
            use_native = False
    if use_native or not torch.cuda.is_available():
        flat = allocate_memory(numel * total, dtype, "cpu", pinned=True)
        blocks = [flat[i * numel:(i + 1) * numel] for i in range(total)]
    else:
        for g in allocate_optimal(total, numel * itemsize):
            chunk = torch.empty(g * numel * itemsize, dtype=torch.uint8).pin_memory().view(dtype)
            blocks.extend(chunk[i * numel:(i + 1) * numel] for i in range(g))

    def nest(level, offset):
        if level == len(shape):
            return blocks[offset]
        stride = 1
        for s in shape[level + 1:]:
            stride *= s
        return [nest(level + 1, offset + i * stride) for i in range(shape[level])]

    return nest(0, 0)


# ------------------------------------------------- locked-tensor manager
# address -> (ctypes buffer, "cuda" | "host"); keeps the mapping alive until freed
_LOCKED: dict = {}


def new_cpu_locked_tensor(numel: int, dtype: torch.dtype) -> torch.Tensor:
    """Exact-size page-locked CPU tensor owned by the native pool.

    With a CUDA context the memory comes from ``cudaHostAlloc`` (portable, so
    every stream can DMA from it); without one it is ``posix_memalign`` +
    ``mlock`` from the host library.  Free it with ``free_cpu_locked_tensor``.
    Counterpart of ``aio_handle.new_cpu_locked_tensor``
    (flextrain/ops/csrc/aio/py_lib/deepspeed_pin_tensor.cpp:23-44)."""
    import ctypes
    from ..ops import native
    from ..utils import distributed as dist
    nbytes = max(1, int(numel) * torch.empty((), dtype=dtype).element_size())
    if dist.is_cuda():
        lib = native.cuda_lib()
        lib.ft_pinned_alloc.restype = ctypes.c_void_p
        addr, kind = lib.ft_pinned_alloc(ctypes.c_size_t(nbytes)), "cuda"
    else:
        lib = native.host_lib()
        lib.ft_locked_alloc.restype = ctypes.c_void_p
        lib.ft_locked_alloc.argtypes = [ctypes.c_size_t, ctypes.c_void_p]
        addr, kind = lib.ft_locked_alloc(nbytes, None), "host"
    if not addr:
        raise MemoryError(f"page-locked allocation of {nbytes} bytes failed")
    buf = (ctypes.c_uint8 * nbytes).from_address(addr)
    _LOCKED[addr] = (buf, kind)
    return torch.frombuffer(buf, dtype=torch.uint8, count=nbytes).view(dtype)[:numel]


def is_cpu_locked_tensor(t: torch.Tensor) -> bool:
    return t.data_ptr() in _LOCKED


def free_cpu_locked_tensor(t: torch.Tensor) -> None:
    """Return a tensor from ``new_cpu_locked_tensor`` to the system.  The caller
    must not touch ``t`` (or views of it) afterwards."""
    import ctypes
    from ..ops import native
    addr = t.data_ptr()
    entry = _LOCKED.pop(addr, None)
    if entry is None:
        raise ValueError("tensor was not allocated by new_cpu_locked_tensor")
    _buf, kind = entry
    if kind == "cuda":
        lib = native.cuda_lib()
        lib.ft_pinned_free.argtypes = [ctypes.c_void_p]
        rc = lib.ft_pinned_free(addr)
    else:
        lib = native.host_lib()
        lib.ft_locked_free.argtypes = [ctypes.c_void_p]
        rc = lib.ft_locked_free(addr)
    if rc != 0:
        raise RuntimeError(f"freeing page-locked memory failed with {rc}")


def host_memcpy(dst: torch.Tensor, src: torch.Tensor, threads: int = 0) -> torch.Tensor:
    """``dst.copy_(src)`` for contiguous CPU tensors of equal byte size, done by
    the native multi-threaded copy with non-temporal stores (``ft_host_memcpy``;
    the reference's counterpart is ``deepspeed_memcpy``,
    flextrain/ops/csrc/aio/py_lib/deepspeed_py_copy.cpp:113-135)."""
    import ctypes
    from ..ops import native
    if dst.device.type != "cpu" or src.device.type != "cpu":
        raise ValueError("host_memcpy copies between CPU tensors")
    if not (dst.is_contiguous() and src.is_contiguous()):
        raise ValueError("host_memcpy needs contiguous tensors")
    nbytes = dst.numel() * dst.element_size()
    if nbytes != src.numel() * src.element_size():
        raise ValueError("host_memcpy needs tensors of equal byte size")
    lib = native.host_lib()
    lib.ft_host_memcpy.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
    rc = lib.ft_host_memcpy(dst.data_ptr(), src.data_ptr(), nbytes, int(threads))
    if rc != 0:
        raise RuntimeError("ft_host_memcpy rejected its arguments (overlapping ranges?)")
    return dst
