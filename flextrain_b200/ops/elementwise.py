"""Small streaming ops the engine itself issues (not the model): gradient
accumulation into a wide buffer, casts and flat copies.

They replace the ATen calls of flextrain/memory/coordinator/optimizer.py:771-777
(``gradacc += grads`` followed by ``zero_``) with one pass.  CUDA tensors go to
the sm_100a kernels; CPU tensors (gloo backend) use the same math in PyTorch.
"""
from __future__ import annotations

import torch

from .native import cuda_lib, dtype_code, ptr, stream_handle


def accumulate_and_zero(acc: torch.Tensor, src: torch.Tensor):
    """``acc += src`` (acc wider or equal dtype), then ``src = 0``; one read of
    ``src``, one read-modify-write of ``acc``."""
    if acc.numel() != src.numel():
        raise ValueError("accumulate_and_zero: size mismatch")
    if acc.is_cuda:
        rc = cuda_lib().ft_accumulate_zero(ptr(acc), dtype_code(acc.dtype), ptr(src),
                                           dtype_code(src.dtype), acc.numel(), stream_handle())
        if rc != 0:
            raise RuntimeError(f"ft_accumulate_zero failed with CUDA error {rc}")
        return
    acc.add_(src.to(acc.dtype))
    src.zero_()


def cast_copy(dst: torch.Tensor, src: torch.Tensor):
    """``dst = (dst.dtype) src`` over flat device tensors."""
    if dst.numel() != src.numel():
        raise ValueError("cast_copy: size mismatch")
    if dst.is_cuda and src.is_cuda:
        rc = cuda_lib().ft_cast_copy(ptr(dst), dtype_code(dst.dtype), ptr(src),
                                     dtype_code(src.dtype), dst.numel(), stream_handle())
        if rc != 0:
            raise RuntimeError(f"ft_cast_copy failed with CUDA error {rc}")
        return
    dst.copy_(src)
