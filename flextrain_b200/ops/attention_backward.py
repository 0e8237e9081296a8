"""Backward of the native causal attention (``ft_attn_bwd``)."""
from __future__ import annotations

import torch

from .native import dtype_code, ptr, stream_handle


def attention_backward(q, k, v, o, lse, do, scale, out=None, trace=None):
    """Gradients (dq, dk, dv) for ``[B,S,H,D]`` inputs with unit inner stride and
    adjacent heads (the tensors the forward saved).  ``out`` may supply
    pre-allocated (dq, dk, dv) views, e.g. into one packed gradient tensor.
    ``trace = (int64 tensor of 5*16*8, cta, first iteration)`` records the timeline
    of one CTA (bf16, head size 128; see ``benchmarks/attn_timeline.py``)."""
    from .attention_native import _lib
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    do = do if (do.stride(3) == 1 and do.stride(2) == D and do.stride(0) == S * do.stride(1)
                and (do.stride(1) * do.element_size()) % 16 == 0) else do.contiguous()
    if out is None:
        dq = torch.empty(B, S, Hq, D, dtype=q.dtype, device=q.device)
        dk = torch.empty(B, S, Hkv, D, dtype=q.dtype, device=q.device)
        dv = torch.empty(B, S, Hkv, D, dtype=q.dtype, device=q.device)
    else:
        dq, dk, dv = out
    delta = torch.empty(B * Hq * S, dtype=torch.float32, device=q.device)
    dq_acc = torch.empty(B * S * Hq * D, dtype=torch.float32, device=q.device)
    args = (ptr(q), q.stride(1), ptr(k), k.stride(1), ptr(v), v.stride(1), ptr(o), ptr(do),
            do.stride(1), ptr(lse), ptr(delta), ptr(dq_acc), ptr(dq), dq.stride(1), ptr(dk),
            dk.stride(1), ptr(dv), dv.stride(1), B, S, Hq, Hkv, D, float(scale),
            dtype_code(q.dtype), stream_handle())
    if trace is None:
        rc = _lib().ft_attn_bwd(*args)
    else:
        buf, cta, it0 = trace
        assert buf.dtype == torch.int64 and buf.numel() >= 5 * 16 * 8 and buf.is_cuda
        rc = _lib().ft_attn_bwd_traced(*args, ptr(buf), int(cta), int(it0))
    if rc != 0:
        raise RuntimeError(f"ft_attn_bwd failed (code {rc})")
    return dq, dk, dv
