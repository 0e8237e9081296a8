"""Causal grouped-query attention on CUDA tensors.

``FLEXTRAIN_ATTN`` selects the implementation: ``native`` (default) is the
package's own sm_100a kernel pair when the CUDA library exports it;
``sdpa`` calls PyTorch's fused scaled-dot-product attention (a library kernel,
kept as the comparison baseline and as the stand-in while a native kernel for a
head size is missing).
"""
from __future__ import annotations

import math
import os

import torch.nn.functional as F

from .native import cuda_lib


def native_available(head_dim: int) -> bool:
    try:
        lib = cuda_lib()
    except Exception:
        return False
    return hasattr(lib, "ft_attn_fwd") and head_dim in (64, 128)


def _sdpa(q, k, v, scale):
    qh, kh, vh = (t.permute(0, 2, 1, 3) for t in (q, k, v))
    out = F.scaled_dot_product_attention(qh, kh, vh, is_causal=True, scale=scale,
                                         enable_gqa=kh.shape[1] != qh.shape[1])
    return out.permute(0, 2, 1, 3)


def causal_attention(q, k, v, scale=None):
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    impl = os.environ.get("FLEXTRAIN_ATTN", "native")
    if impl == "native" and native_available(q.shape[-1]):
        from .attention_native import attention_native
        return attention_native(q, k, v, scale)
    return _sdpa(q, k, v, scale)
