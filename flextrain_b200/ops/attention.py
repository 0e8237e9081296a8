"""Causal grouped-query attention on CUDA tensors.

``FLEXTRAIN_ATTN`` selects the implementation: ``native`` (default) is the
package's own sm_100a kernel pair when the CUDA library exports it;
``sdpa`` calls PyTorch's fused scaled-dot-product attention (a library kernel,
kept as the comparison baseline).  A head size the native kernels do not cover
raises; it does not fall back.
"""
from __future__ import annotations

import math
import os

import torch.nn.functional as F

from .native import cuda_lib


def native_available(head_dim: int) -> bool:
    """Whether the package's own kernels cover this head size.  A missing CUDA library raises
    (a GPU run must never end up on eager PyTorch without being asked to)."""
    return hasattr(cuda_lib(), "ft_attn_fwd") and head_dim in (64, 128)


def _sdpa(q, k, v, scale):
    qh, kh, vh = (t.permute(0, 2, 1, 3) for t in (q, k, v))
    out = F.scaled_dot_product_attention(qh, kh, vh, is_causal=True, scale=scale,
                                         enable_gqa=kh.shape[1] != qh.shape[1])
    return out.permute(0, 2, 1, 3)


def causal_attention(q, k, v, scale=None):
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    impl = os.environ.get("FLEXTRAIN_ATTN", "native")
    if impl == "sdpa":
        return _sdpa(q, k, v, scale)
    if not native_available(q.shape[-1]):
        raise NotImplementedError(
            f"no native attention kernel for head size {q.shape[-1]} (64 and 128 are built); set "
            "FLEXTRAIN_ATTN=sdpa to run PyTorch's scaled_dot_product_attention instead")
    from .attention_native import attention_native
    return attention_native(q, k, v, scale)
