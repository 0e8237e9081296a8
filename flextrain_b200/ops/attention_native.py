"""Autograd binding of the native causal attention kernels
(``csrc/kernels/attention_fwd.cuh`` / ``attention_bwd.cuh``).

``q``, ``k``, ``v`` may be strided views into one packed QKV tensor (unit stride
inside a head, heads adjacent); nothing is copied on the way in.
"""
from __future__ import annotations

import torch

from .native import cuda_lib, dtype_code, ptr, stream_handle

_DECLARED = False


def _lib():
    global _DECLARED
    lib = cuda_lib()
    if not _DECLARED:
        from ctypes import c_float, c_int, c_int64, c_void_p
        lib.ft_attn_fwd.argtypes = [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p,
                                    c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p]
        if hasattr(lib, "ft_attn_fwd_traced"):
            lib.ft_attn_fwd_traced.argtypes = list(lib.ft_attn_fwd.argtypes) + [c_void_p, c_int, c_int]
            lib.ft_attn_fwd_traced.restype = c_int
        if hasattr(lib, "ft_attn_bwd"):
            lib.ft_attn_bwd.argtypes = [c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_void_p,
                                        c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
                                        c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_int,
                                        c_int, c_float, c_int, c_void_p]
        if hasattr(lib, "ft_attn_bwd_traced"):
            lib.ft_attn_bwd_traced.argtypes = list(lib.ft_attn_bwd.argtypes) + [c_void_p, c_int, c_int]
            lib.ft_attn_bwd_traced.restype = c_int
        _DECLARED = True
    return lib


def _rows(t: torch.Tensor):
    """(tensor usable by the kernel, token stride) for a [B, S, H, D] tensor."""
    B, S, H, D = t.shape
    ok = t.stride(3) == 1 and t.stride(2) == D and t.stride(0) == S * t.stride(1) \
        and (t.stride(1) * t.element_size()) % 16 == 0 and t.data_ptr() % 16 == 0
    if not ok:
        t = t.contiguous()
    return t, t.stride(1)


def attention_forward(q, k, v, scale, trace=None):
    """``trace = (int64 tensor of 3*8*8, cta, first K/V block)`` records the timeline of one CTA
    (bf16, head size 128; see ``benchmarks/attn_timeline.py``)."""
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    q, qs = _rows(q)
    k, ks = _rows(k)
    v, vs = _rows(v)
    o = torch.empty(B, S, Hq, D, dtype=q.dtype, device=q.device)
    lse = torch.empty(B, Hq, S, dtype=torch.float32, device=q.device)
    args = (ptr(q), qs, ptr(k), ks, ptr(v), vs, ptr(o), ptr(lse), B, S, Hq, Hkv, D,
            float(scale), dtype_code(q.dtype), stream_handle())
    if trace is None:
        rc = _lib().ft_attn_fwd(*args)
    else:
        buf, cta, it0 = trace
        assert buf.dtype == torch.int64 and buf.numel() >= 3 * 8 * 8 and buf.is_cuda
        rc = _lib().ft_attn_fwd_traced(*args, ptr(buf), int(cta), int(it0))
    if rc != 0:
        raise RuntimeError(f"ft_attn_fwd failed (code {rc})")
    return o, lse, (q, k, v)


class _Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale):
        o, lse, (qc, kc, vc) = attention_forward(q, k, v, scale)
        ctx.save_for_backward(qc, kc, vc, o, lse)
        ctx.scale = scale
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        from .attention_backward import attention_backward
        dq, dk, dv = attention_backward(q, k, v, o, lse, do, ctx.scale)
        return dq, dk, dv, None


def attention_native(q, k, v, scale):
    return _Attention.apply(q, k, v, scale)


class _PackedAttention(torch.autograd.Function):
    """Attention over a packed ``qkv [B, S, (Hq + 2*Hkv) * D]`` tensor whose q and
    k heads are already rotated.  The backward writes dq, dk and dv straight into
    one packed gradient tensor, so no slice gradients are materialised."""

    @staticmethod
    def forward(ctx, qkv, hq, hkv, d, scale):
        B, S, _ = qkv.shape
        q = qkv[..., : hq * d].unflatten(-1, (hq, d))
        k = qkv[..., hq * d:(hq + hkv) * d].unflatten(-1, (hkv, d))
        v = qkv[..., (hq + hkv) * d:].unflatten(-1, (hkv, d))
        o, lse, _ = attention_forward(q, k, v, scale)
        ctx.save_for_backward(qkv, o, lse)
        ctx.meta = (hq, hkv, d, scale)
        return o.view(B, S, hq * d)

    @staticmethod
    def backward(ctx, do):
        qkv, o, lse = ctx.saved_tensors
        hq, hkv, d, scale = ctx.meta
        B, S, _ = qkv.shape
        from .attention_backward import attention_backward
        q = qkv[..., : hq * d].unflatten(-1, (hq, d))
        k = qkv[..., hq * d:(hq + hkv) * d].unflatten(-1, (hkv, d))
        v = qkv[..., (hq + hkv) * d:].unflatten(-1, (hkv, d))
        dqkv = torch.empty_like(qkv)
        outs = (dqkv[..., : hq * d].unflatten(-1, (hq, d)),
                dqkv[..., hq * d:(hq + hkv) * d].unflatten(-1, (hkv, d)),
                dqkv[..., (hq + hkv) * d:].unflatten(-1, (hkv, d)))
        attention_backward(q, k, v, o, lse, do.reshape(B, S, hq, d), scale, out=outs)
        return dqkv, None, None, None, None


def attention_packed(qkv, hq, hkv, d, scale):
    return _PackedAttention.apply(qkv, hq, hkv, d, scale)
