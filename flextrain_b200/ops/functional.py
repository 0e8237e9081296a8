"""Model ops as the Llama and GPT blocks call them.

CUDA tensors are routed to the hand-written sm_100a kernels (``cuda_ops``);
a missing CUDA library raises instead of silently running eager PyTorch.  CPU
tensors use the plain PyTorch statements in ``reference`` (gloo backend).
"""
from __future__ import annotations

import os

import torch

from . import reference as ref


def _cuda(t: torch.Tensor) -> bool:
    return t.is_cuda


def linear(x, w):
    if _cuda(x):
        from . import cuda_ops
        return cuda_ops.linear(x, w)
    return ref.linear(x, w)


def linear_add(x, w, res):
    """``res + linear(x, w)``; on CUDA the addition runs in the epilogue of the GEMM."""
    if _cuda(x):
        from . import cuda_ops
        return cuda_ops.linear_add(x, w, res)
    return res + ref.linear(x, w)


def rmsnorm(x, weight, eps):
    if _cuda(x):
        from . import cuda_ops
        # row-resident kernels (each row read once): 0.70-0.72 of the HBM copy rate forward,
        # 0.54-0.60 backward at hidden 5120 / 8192, against 0.37 / 0.25 for the two-pass
        # kernels, which remain for hidden sizes the row kernels do not cover
        if cuda_ops.norm_rows_supported(x.shape[-1]) and os.environ.get("FLEXTRAIN_RMSNORM", "rows") == "rows":
            return cuda_ops.rmsnorm_rows(x, weight, eps)
        return cuda_ops.rmsnorm(x, weight, eps)
    return ref.rmsnorm(x, weight, eps)


def add_rmsnorm(x, r, weight, eps):
    """``s = x + r`` and ``rmsnorm(s) * weight`` in one pass over the rows; returns ``(s, y)``.
    The residual add of a transformer block and the norm that follows it (forward), and the
    sum of the two gradient branches that meet at ``s`` (backward), cost no pass of their own."""
    if _cuda(x):
        from . import cuda_ops
        if cuda_ops.norm_rows_supported(x.shape[-1]) and os.environ.get("FLEXTRAIN_RMSNORM", "rows") == "rows":
            return cuda_ops.add_rmsnorm(x, r, weight, eps)
        s = x + r
        return s, cuda_ops.rmsnorm(s, weight, eps)
    s = x + r
    return s, ref.rmsnorm(s, weight, eps)


def gpt_native_elementwise() -> bool:
    """Whether CUDA tensors take the package's LayerNorm / bias / GELU kernels (default) or
    the ATen ones (``FLEXTRAIN_GPT_ELEMENTWISE=aten``, the comparison arm of
    ``benchmarks/elementwise_bench.py``).  GEMMs and attention are native either way."""
    return os.environ.get("FLEXTRAIN_GPT_ELEMENTWISE", "native") == "native"


def layernorm(x, weight, bias, eps):
    if _cuda(x):
        if gpt_native_elementwise():
            from . import cuda_ops
            return cuda_ops.layernorm(x, weight, bias, eps)
        return torch.nn.functional.layer_norm(x, (x.shape[-1],), weight, bias, eps)
    return ref.layernorm(x, weight, bias, eps)


def bias_add(x, bias):
    """``x + bias`` over the last dimension (in place on CUDA with the native kernels)."""
    if _cuda(x):
        if gpt_native_elementwise():
            from . import cuda_ops
            return cuda_ops.bias_add(x, bias)
        return x + bias
    return ref.bias_add(x, bias)


def bias_gelu(x, bias):
    if _cuda(x):
        if gpt_native_elementwise():
            from . import cuda_ops
            return cuda_ops.bias_gelu(x, bias)
        return torch.nn.functional.gelu(x + bias, approximate="tanh")
    return ref.bias_gelu(x, bias)


def rope(x, cos, sin):
    if _cuda(x):
        from . import cuda_ops
        return cuda_ops.rope(x, cos, sin)
    return ref.rope(x, cos, sin)


def rope_heads_inplace(x, cos, sin, heads, d):
    from . import cuda_ops
    return cuda_ops.rope_heads_inplace(x, cos, sin, heads, d)


def attention_packed(qkv, hq, hkv, d, scale=None):
    """Causal attention over a packed, already rotated ``qkv [B, S, (hq+2*hkv)*d]``
    with the native kernels; None when they do not cover this head size or
    ``FLEXTRAIN_ATTN=sdpa`` asks for the library path."""
    import math
    import os
    from .attention import native_available
    if os.environ.get("FLEXTRAIN_ATTN", "native") == "sdpa" or not native_available(d):
        return None
    from .attention_native import attention_packed as impl
    return impl(qkv, hq, hkv, d, scale if scale is not None else 1.0 / math.sqrt(d))


def swiglu(gate_up):
    if _cuda(gate_up):
        from . import cuda_ops
        return cuda_ops.swiglu(gate_up)
    return ref.swiglu(gate_up)


def linear_swiglu(x, w_gate_up):
    """``swiglu(linear(x, w_gate_up))``.  On CUDA the activation runs in the epilogue of the
    projection GEMM where that measured faster: always when no gradient is recorded (the
    [M, 2F] intermediate is then never written: 1.4 % to 20 % less time at the 13B / 70B / 7B
    shapes), and with a gradient for hidden sizes from 5120 (1.4 % / 3.3 % at 13B / 70B; at
    4096 the fused kernel's backward path was 12 % slower than two kernels).
    ``FLEXTRAIN_SWIGLU=epilogue|separate`` forces one form."""
    if _cuda(x):
        mode = os.environ.get("FLEXTRAIN_SWIGLU", "auto")
        needs_grad = torch.is_grad_enabled() and (x.requires_grad or w_gate_up.requires_grad)
        if mode == "epilogue" or (mode == "auto" and (not needs_grad or x.shape[-1] >= 5120)):
            from . import cuda_ops
            return cuda_ops.linear_swiglu(x, w_gate_up)
    return swiglu(linear(x, w_gate_up))


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
