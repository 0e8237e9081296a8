"""ctypes access to the two native libraries of the package.

``host_lib()``  - AVX-512 Adam, NVMe engine, host copies (built with g++).
``cuda_lib()``  - every sm_100a kernel, the pinned pool and the peer-memory
                  helpers (built with nvcc for ``sm_100a``).

Tensors cross the boundary as raw addresses (``tensor.data_ptr()``) plus
element counts; CUDA kernels additionally take the caller's stream handle.
ctypes drops the GIL for the duration of each call, which is what lets the host
Adam run in a worker thread beside the Python thread that feeds the GPU.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_int64, c_void_p
from typing import Optional

import torch

from .op_builder import BuildError, CudaOpsBuilder, HostOpsBuilder

DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}

_HOST: Optional[ctypes.CDLL] = None
_CUDA: Optional[ctypes.CDLL] = None


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return DTYPE_CODE[dtype]
    except KeyError:
        raise TypeError(f"native kernels support fp32/bf16/fp16, not {dtype}") from None


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def host_lib() -> ctypes.CDLL:
    global _HOST
    if _HOST is None:
        lib = HostOpsBuilder().load()
        lib.ft_adam_simd_level.restype = c_int
        lib.ft_adam_create.argtypes = [c_int, c_float, c_float, c_float, c_float, c_float, c_int]
        lib.ft_adam_destroy.argtypes = [c_int]
        lib.ft_adam_update.argtypes = [
            c_int64, c_float, c_float, c_float, c_float, c_float, c_int, c_int, c_float,
            c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int64, c_void_p, c_int, c_int, c_int]
        lib.ft_adam_update.restype = c_int
        lib.ft_has_nonfinite.argtypes = [c_void_p, c_int, c_int64, c_int]
        lib.ft_cast_from_f32.argtypes = [c_void_p, c_void_p, c_int, c_int64, c_int]
        lib.ft_cast_to_f32.argtypes = [c_void_p, c_int, c_void_p, c_int64, c_int]
        lib.ft_host_memcpy.argtypes = [c_void_p, c_void_p, ctypes.c_size_t, c_int]
        _HOST = lib
    return _HOST


def cuda_lib() -> ctypes.CDLL:
    """Loads the CUDA library; raises if it is missing so that a GPU run can
    never silently fall back to eager PyTorch math."""
    global _CUDA
    if _CUDA is None:
        lib = CudaOpsBuilder().load()
        from . import _cuda_sigs
        _cuda_sigs.declare(lib)
        _CUDA = lib
    return _CUDA


def cuda_lib_available() -> bool:
    try:
        cuda_lib()
        return True
    except (BuildError, OSError):
        return False


def stream_handle(stream: Optional["torch.cuda.Stream"] = None) -> int:
    s = stream if stream is not None else torch.cuda.current_stream()
    return s.cuda_stream
