"""Model ops as the Llama blocks call them.

CUDA tensors are routed to the hand-written sm_100a kernels (``cuda_ops``);
a missing CUDA library raises instead of silently running eager PyTorch.  CPU
tensors use the plain PyTorch statements in ``reference`` (gloo backend).
"""
from __future__ import annotations

import torch

from . import reference as ref


def _cuda(t: torch.Tensor) -> bool:
    return t.is_cuda


def linear(x, w):
    if _cuda(x):
        from . import cuda_ops
        return cuda_ops.linear(x, w)
    return ref.linear(x, w)


def rmsnorm(x, weight, eps):
    if _cuda(x):
        from . import cuda_ops
        return cuda_ops.rmsnorm(x, weight, eps)
    return ref.rmsnorm(x, weight, eps)


def rope(x, cos, sin):
    if _cuda(x):
        from . import cuda_ops
        return cuda_ops.rope(x, cos, sin)
    return ref.rope(x, cos, sin)


def rope_heads_inplace(x, cos, sin, heads, d):
    from . import cuda_ops
    return cuda_ops.rope_heads_inplace(x, cos, sin, heads, d)


def swiglu(gate_up):
    if _cuda(gate_up):
        from . import cuda_ops
        return cuda_ops.swiglu(gate_up)
    return ref.swiglu(gate_up)


def causal_attention(q, k, v, scale=None):
    if _cuda(q):
        from . import cuda_ops
        return cuda_ops.causal_attention(q, k, v, scale)
    return ref.causal_attention(q, k, v, scale)


def linear_cross_entropy(hidden, weight, labels, ignore_index=-100):
    if _cuda(hidden):
        from . import cuda_ops
        return cuda_ops.linear_cross_entropy(hidden, weight, labels, ignore_index)
    return ref.linear_cross_entropy(hidden, weight, labels, ignore_index)


rope_tables = ref.rope_tables
