"""Autograd bindings of the hand-written sm_100a kernels.

Each op is a ``torch.autograd.Function`` whose forward and backward launch the
kernels of ``csrc/kernels`` on the current CUDA stream.  There is no eager
fallback here: if the CUDA library is missing these raise.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from .native import cuda_lib, dtype_code, ptr, stream_handle


def _check(rc: int, what: str):
    if rc != 0:
        raise RuntimeError(f"{what} failed (code {rc})")


# --------------------------------------------------------------------- GEMM
def gemm(a: torch.Tensor, a_mn: bool, b: torch.Tensor, b_mn: bool, m: int, n: int, k: int,
         out: Optional[torch.Tensor] = None, accumulate: bool = False,
         out_dtype: Optional[torch.dtype] = None, add: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[m, n] (+)= sum_k A(m, k) B(n, k)`` on the tcgen05 tensor cores.
    ``a`` is stored ``[m, k]`` (``a_mn=False``) or ``[k, m]`` (``a_mn=True``);
    ``b`` is stored ``[n, k]`` or ``[k, n]`` likewise.  Inputs are 2-D with unit
    inner stride.  ``add`` (``[m, n]``, the type of ``out``, unit inner stride) is added
    to the product in the epilogue: ``out = A B^T + add``."""
    if a.dtype != b.dtype or a.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError("gemm operands must both be bf16 or both fp16")
    if a.stride(-1) != 1 or b.stride(-1) != 1:
        raise ValueError("gemm operands need unit inner stride")
    if out is None:
        out = torch.empty(m, n, dtype=out_dtype or a.dtype, device=a.device)
        accumulate = False
    if add is not None:
        if add.shape != (m, n) or add.dtype != out.dtype or add.stride(-1) != 1:
            raise ValueError("gemm: `add` must be [m, n] of the output's type with unit inner stride")
        rc = cuda_lib().ft_gemm_add(ptr(a), int(a_mn), a.stride(0), ptr(b), int(b_mn), b.stride(0), ptr(out),
                                    out.stride(0), dtype_code(out.dtype), 1, ptr(add), add.stride(0), m, n, k,
                                    dtype_code(a.dtype), stream_handle())
        _check(rc, "ft_gemm_add")
        return out
    rc = cuda_lib().ft_gemm(ptr(a), int(a_mn), a.stride(0), ptr(b), int(b_mn), b.stride(0), ptr(out),
                            out.stride(0), dtype_code(out.dtype), int(accumulate), m, n, k,
                            dtype_code(a.dtype), stream_handle())
    _check(rc, "ft_gemm")
    return out


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        k = x.shape[-1]
        x2 = x.reshape(-1, k)
        if x2.stride(-1) != 1 or (x2.stride(0) * x2.element_size()) % 16:
            x2 = x2.contiguous()
        n = w.shape[0]
        y = torch.empty(*x.shape[:-1], n, dtype=x.dtype, device=x.device)
        pending = getattr(w, "_ft_gather", None)
        if pending is not None:
            # the rows of this weight that other ranks own are not in the gathered buffer yet:
            # one kernel brings them in over NVLink and multiplies (csrc/comm/ag_gemm.cu)
            if pending.covers(x2.shape[0], k):
                pending.run(x2, y.view(-1, n))
            else:
                pending.complete_without_product()
                gemm(x2, False, w, False, x2.shape[0], n, k, out=y.view(-1, n))
        else:
            gemm(x2, False, w, False, x2.shape[0], n, k, out=y.view(-1, n))
        ctx.save_for_backward(x2, w)
        ctx.x_shape = x.shape
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        n, k = w.shape
        dy2 = dy.reshape(-1, n)
        if dy2.stride(-1) != 1 or (dy2.stride(0) * dy2.element_size()) % 16:
            dy2 = dy2.contiguous()
        m = dy2.shape[0]
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, False, w, True, m, k, n).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            g = w.grad
            if g is not None and g.shape == w.shape and g.is_contiguous() and g.dtype == w.dtype:
                # accumulate straight into the engine's gradient buffer
                gemm(dy2, True, x2, True, n, k, m, out=g, accumulate=True)
            else:
                dw = gemm(dy2, True, x2, True, n, k, m)
        return dx, dw


def linear(x, w):
    return _Linear.apply(x, w)


class _LinearAdd(torch.autograd.Function):
    """``res + x w^T`` with the addition in the GEMM epilogue (one read of ``res`` instead of an
    element-wise pass over two tensors).  The gradient of ``res`` is the output gradient itself."""

    @staticmethod
    def forward(ctx, x, w, res):
        k = x.shape[-1]
        x2 = x.reshape(-1, k)
        if x2.stride(-1) != 1 or (x2.stride(0) * x2.element_size()) % 16:
            x2 = x2.contiguous()
        n = w.shape[0]
        r2 = res.reshape(-1, n)
        if r2.stride(-1) != 1:
            r2 = r2.contiguous()
        y = torch.empty(*x.shape[:-1], n, dtype=x.dtype, device=x.device)
        pending = getattr(w, "_ft_gather", None)
        if pending is not None:
            pending.complete_without_product()
        gemm(x2, False, w, False, x2.shape[0], n, k, out=y.view(-1, n), add=r2)
        ctx.save_for_backward(x2, w)
        ctx.x_shape = x.shape
        return y

    @staticmethod
    def backward(ctx, dy):
        dx, dw = _Linear.backward(ctx, dy)
        return dx, dw, (dy if ctx.needs_input_grad[2] else None)


def linear_add(x, w, res):
    return _LinearAdd.apply(x, w, res)


# ------------------------------------------------------------------ RMSNorm
class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        h = x.shape[-1]
        x2 = x.reshape(-1, h).contiguous()
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        inv = torch.empty(rows, dtype=torch.float32, device=x.device)
        _check(cuda_lib().ft_rmsnorm_fwd(ptr(x2), ptr(w), ptr(y), ptr(inv), rows, h, float(eps),
                                         dtype_code(x.dtype), stream_handle()), "ft_rmsnorm_fwd")
        ctx.save_for_backward(x2, w, inv)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w, inv = ctx.saved_tensors
        rows, h = x2.shape
        dy2 = dy.reshape(rows, h).contiguous()
        dx = torch.empty_like(x2)
        dw = torch.empty_like(w)
        lib = cuda_lib()
        part = torch.empty(lib.ft_rmsnorm_bwd_parts() * h, dtype=torch.float32, device=x2.device)
        _check(lib.ft_rmsnorm_bwd(ptr(x2), ptr(w), ptr(dy2), ptr(inv), ptr(dx), ptr(dw), ptr(part), rows,
                                  h, dtype_code(x2.dtype), stream_handle()), "ft_rmsnorm_bwd")
        return dx.view(dy.shape), dw, None


def rmsnorm(x, w, eps):
    return _RMSNorm.apply(x, w, eps)


class _Norm(torch.autograd.Function):
    """LayerNorm (``b`` given) or RMSNorm (``b`` None) through the register-resident
    row kernels (``ft_norm_fwd`` / ``ft_norm_bwd``)."""

    @staticmethod
    def forward(ctx, x, w, b, eps):
        h = x.shape[-1]
        x2 = x.reshape(-1, h).contiguous()
        rows = x2.shape[0]
        ln = b is not None
        y = torch.empty_like(x2)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device) if ln else None
        _check(cuda_lib().ft_norm_fwd(ptr(x2), ptr(w), ptr(b) if ln else None, ptr(y),
                                      ptr(mean) if ln else None, ptr(rstd), rows, h, float(eps), int(ln),
                                      dtype_code(x.dtype), stream_handle()), "ft_norm_fwd")
        ctx.save_for_backward(x2, w, mean, rstd)
        ctx.ln = ln
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w, mean, rstd = ctx.saved_tensors
        rows, h = x2.shape
        ln = ctx.ln
        dy2 = dy.reshape(rows, h).contiguous()
        dx = torch.empty_like(x2)
        dw = torch.empty_like(w)
        db = torch.empty_like(w) if ln else None
        lib = cuda_lib()
        parts = lib.ft_norm_bwd_parts(rows, h)
        part = torch.empty((2 if ln else 1) * parts * h, dtype=torch.float32, device=x2.device)
        db_part = part[parts * h:] if ln else None
        _check(lib.ft_norm_bwd(ptr(x2), ptr(w), ptr(dy2), ptr(mean) if ln else None, ptr(rstd), ptr(dx),
                               ptr(dw), ptr(db) if ln else None, ptr(part),
                               ptr(db_part) if ln else None, rows, h, int(ln), dtype_code(x2.dtype),
                               stream_handle()), "ft_norm_bwd")
        return dx.view(dy.shape), dw, db, None


def layernorm(x, w, b, eps):
    return _Norm.apply(x, w, b, eps)


def rmsnorm_rows(x, w, eps):
    """RMSNorm through the same row kernels as ``layernorm`` (each row read once)."""
    return _Norm.apply(x, w, None, eps)


_NORM_MAX_HIDDEN = None


def norm_rows_supported(hidden: int) -> bool:
    """Whether the row-resident norm kernels cover this hidden size (forward and backward)."""
    global _NORM_MAX_HIDDEN
    if _NORM_MAX_HIDDEN is None:
        lib = cuda_lib()
        _NORM_MAX_HIDDEN = min(lib.ft_norm_max_hidden(0), lib.ft_norm_max_hidden(1))
    return hidden % 8 == 0 and 0 < hidden <= _NORM_MAX_HIDDEN


class _AddRMSNorm(torch.autograd.Function):
    """``s = x + r`` and ``y = rmsnorm(s) * w`` in one kernel; the backward adds the gradient
    that arrives at ``s`` from its other consumer (the next residual add) to the gradient through
    the norm inside the norm's backward kernel, so neither direction has an add pass."""

    @staticmethod
    def forward(ctx, x, r, w, eps):
        h = x.shape[-1]
        x2 = x.reshape(-1, h).contiguous()
        r2 = r.reshape(-1, h).contiguous()
        rows = x2.shape[0]
        s = torch.empty_like(x2)
        y = torch.empty_like(x2)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        _check(cuda_lib().ft_add_norm_fwd(ptr(x2), ptr(r2), ptr(s), ptr(w), None, ptr(y), None, ptr(rstd),
                                          rows, h, float(eps), 0, dtype_code(x.dtype), stream_handle()),
               "ft_add_norm_fwd")
        ctx.save_for_backward(s, w, rstd)
        return s.view(x.shape), y.view(x.shape)

    @staticmethod
    def backward(ctx, ds, dy):
        s, w, rstd = ctx.saved_tensors
        rows, h = s.shape
        if dy is None:
            return ds, ds, None, None
        dy2 = dy.reshape(rows, h).contiguous()
        ds2 = ds.reshape(rows, h).contiguous() if ds is not None else None
        dx = torch.empty_like(s)
        dw = torch.empty_like(w)
        lib = cuda_lib()
        parts = lib.ft_norm_bwd_parts(rows, h)
        part = torch.empty(parts * h, dtype=torch.float32, device=s.device)
        _check(lib.ft_add_norm_bwd(ptr(s), ptr(w), ptr(dy2), ptr(ds2), None, ptr(rstd), ptr(dx), ptr(dw),
                                   None, ptr(part), None, rows, h, 0, dtype_code(s.dtype), stream_handle()),
               "ft_add_norm_bwd")
        dx = dx.view(dy.shape)
        return dx, dx, dw, None


def add_rmsnorm(x, r, w, eps):
    return _AddRMSNorm.apply(x, r, w, eps)


class _BiasAct(torch.autograd.Function):
    """``act(x + bias)`` over the last dimension; act 0 adds the bias in place,
    act 1 is the tanh GELU.  The backward produces dx and the bias gradient (column
    sums of dx) in one pass."""

    @staticmethod
    def forward(ctx, x, bias, act):
        n = x.shape[-1]
        x2 = x.reshape(-1, n)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        rows = x2.shape[0]
        in_place = act == 0 and x2.data_ptr() == x.data_ptr()
        y = x2 if in_place else torch.empty_like(x2)
        _check(cuda_lib().ft_bias_act_fwd(ptr(x2), ptr(bias), ptr(y), rows, n, int(act),
                                          dtype_code(x.dtype), stream_handle()), "ft_bias_act_fwd")
        ctx.act = act
        if act == 0:
            ctx.save_for_backward(bias)
        else:
            ctx.save_for_backward(bias, x2)
        if in_place:
            ctx.mark_dirty(x)
            return x
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        act = ctx.act
        bias = ctx.saved_tensors[0]
        n = bias.shape[0]
        dy2 = dy.reshape(-1, n)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        rows = dy2.shape[0]
        lib = cuda_lib()
        parts = lib.ft_bias_act_bwd_parts(rows, n)
        part = torch.empty(parts * n, dtype=torch.float32, device=dy.device)
        dbias = torch.empty_like(bias)
        if act == 0:
            dx2 = dy2
            x_ptr = dx_ptr = None
        else:
            x2 = ctx.saved_tensors[1]
            dx2 = torch.empty_like(dy2)
            x_ptr, dx_ptr = ptr(x2), ptr(dx2)
        _check(lib.ft_bias_act_bwd(ptr(dy2), x_ptr, ptr(bias) if act else None, dx_ptr, ptr(dbias),
                                   ptr(part), rows, n, int(act), 0, dtype_code(dy.dtype),
                                   stream_handle()), "ft_bias_act_bwd")
        return dx2.view(dy.shape), dbias, None


def bias_add(x, bias):
    return _BiasAct.apply(x, bias, 0)


def bias_gelu(x, bias):
    return _BiasAct.apply(x, bias, 1)


# --------------------------------------------------------------------- RoPE
def _rope_launch(x, y, cos, sin, heads, d, seq_len, sign):
    tokens = x.numel() // x.shape[-1] if x.dim() > 1 else 1
    xs = x.reshape(-1, x.shape[-1]) if x.is_contiguous() else x
    tok_stride_x = x.stride(-2) if x.dim() >= 2 else x.shape[-1]
    tok_stride_y = y.stride(-2) if y.dim() >= 2 else y.shape[-1]
    _check(cuda_lib().ft_rope(ptr(x), tok_stride_x, ptr(y), tok_stride_y, ptr(cos), ptr(sin), tokens,
                              heads, d, seq_len, float(sign), dtype_code(x.dtype), stream_handle()),
           "ft_rope")


class _RopeHeads(torch.autograd.Function):
    """Rotate the first ``heads`` heads of every row of ``x`` ``[B, S, W]`` in
    place (rows may be wider than ``heads * d``: the rest is left untouched)."""

    @staticmethod
    def forward(ctx, x, cos, sin, heads, d):
        B, S = x.shape[0], x.shape[1]
        _check(cuda_lib().ft_rope(ptr(x), x.stride(1), ptr(x), x.stride(1), ptr(cos), ptr(sin), B * S,
                                  heads, d, S, 1.0, dtype_code(x.dtype), stream_handle()), "ft_rope")
        ctx.mark_dirty(x)
        ctx.save_for_backward(cos, sin)
        ctx.meta = (heads, d)
        return x

    @staticmethod
    def backward(ctx, dy):
        cos, sin = ctx.saved_tensors
        heads, d = ctx.meta
        dy = dy.contiguous()
        B, S = dy.shape[0], dy.shape[1]
        _check(cuda_lib().ft_rope(ptr(dy), dy.stride(1), ptr(dy), dy.stride(1), ptr(cos), ptr(sin), B * S,
                                  heads, d, S, -1.0, dtype_code(dy.dtype), stream_handle()), "ft_rope")
        return dy, None, None, None, None


def rope_heads_inplace(x, cos, sin, heads, d):
    """In-place rotary embedding of the leading ``heads`` heads of ``x [B, S, W]``."""
    if x.stride(2) != 1 or x.stride(0) != x.shape[1] * x.stride(1):
        raise ValueError("rope_heads_inplace needs a [B, S, W] tensor with contiguous rows")
    return _RopeHeads.apply(x, cos.float().contiguous(), sin.float().contiguous(), heads, d)


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin):
        B, S, H, D = x.shape
        xc = x if (x.stride(3) == 1 and x.stride(2) == D and x.stride(0) == S * x.stride(1)) \
            else x.contiguous()
        y = torch.empty(B, S, H, D, dtype=x.dtype, device=x.device)
        _check(cuda_lib().ft_rope(ptr(xc), xc.stride(1), ptr(y), y.stride(1), ptr(cos), ptr(sin), B * S,
                                  H, D, S, 1.0, dtype_code(x.dtype), stream_handle()), "ft_rope")
        ctx.save_for_backward(cos, sin)
        return y

    @staticmethod
    def backward(ctx, dy):
        cos, sin = ctx.saved_tensors
        dy = dy.contiguous()
        B, S, H, D = dy.shape
        dx = torch.empty_like(dy)
        _check(cuda_lib().ft_rope(ptr(dy), dy.stride(1), ptr(dx), dx.stride(1), ptr(cos), ptr(sin), B * S,
                                  H, D, S, -1.0, dtype_code(dy.dtype), stream_handle()), "ft_rope")
        return dx, None, None


def rope(x, cos, sin):
    return _Rope.apply(x, cos.float().contiguous(), sin.float().contiguous())


# ------------------------------------------------------------------- SwiGLU
class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        f = gu.shape[-1] // 2
        g2 = gu.reshape(-1, 2 * f).contiguous()
        out = torch.empty(g2.shape[0], f, dtype=gu.dtype, device=gu.device)
        _check(cuda_lib().ft_swiglu_fwd(ptr(g2), ptr(out), g2.shape[0], f, dtype_code(gu.dtype),
                                        stream_handle()), "ft_swiglu_fwd")
        ctx.save_for_backward(g2)
        return out.view(*gu.shape[:-1], f)

    @staticmethod
    def backward(ctx, dout):
        (g2,) = ctx.saved_tensors
        rows, f2 = g2.shape
        d2 = dout.reshape(rows, f2 // 2).contiguous()
        dgu = torch.empty_like(g2)
        _check(cuda_lib().ft_swiglu_bwd(ptr(g2), ptr(d2), ptr(dgu), rows, f2 // 2, dtype_code(g2.dtype),
                                        stream_handle()), "ft_swiglu_bwd")
        return dgu.view(*dout.shape[:-1], f2)


def swiglu(gate_up):
    return _SwiGLU.apply(gate_up)


class _LinearSwiGLU(torch.autograd.Function):
    """``swiglu(x @ w.T)`` for ``w = [w_gate ; w_up]`` with the activation in the
    GEMM's epilogue.  The ``[rows, 2F]`` projection is materialised only when a
    backward pass will need it (it is stored from the epilogue's registers, never
    read back in the forward)."""

    @staticmethod
    def forward(ctx, x, w):
        k = x.shape[-1]
        x2 = x.reshape(-1, k)
        if x2.stride(-1) != 1 or (x2.stride(0) * x2.element_size()) % 16:
            x2 = x2.contiguous()
        rows, f = x2.shape[0], w.shape[0] // 2
        need_gu = any(ctx.needs_input_grad[:2])
        act = torch.empty(rows, f, dtype=x.dtype, device=x.device)
        gu = torch.empty(rows, 2 * f, dtype=x.dtype, device=x.device) if need_gu else None
        lib = cuda_lib()
        rc = lib.ft_gemm_swiglu(ptr(x2), x2.stride(0), ptr(w), w.stride(0), ptr(act), f, ptr(gu), 2 * f,
                                rows, f, k, dtype_code(x.dtype), stream_handle())
        if rc == -4:                                   # shape outside the fused kernel: two steps
            gu = torch.empty(rows, 2 * f, dtype=x.dtype, device=x.device)
            gemm(x2, False, w, False, rows, 2 * f, k, out=gu)
            _check(lib.ft_swiglu_fwd(ptr(gu), ptr(act), rows, f, dtype_code(x.dtype), stream_handle()),
                   "ft_swiglu_fwd")
            if not need_gu:
                gu = None
        else:
            _check(rc, "ft_gemm_swiglu")
        ctx.save_for_backward(x2, w, gu)
        ctx.x_shape = x.shape
        return act.view(*x.shape[:-1], f)

    @staticmethod
    def backward(ctx, dact):
        x2, w, gu = ctx.saved_tensors
        rows, f2 = gu.shape
        k = w.shape[1]
        d2 = dact.reshape(rows, f2 // 2).contiguous()
        dgu = torch.empty_like(gu)
        _check(cuda_lib().ft_swiglu_bwd(ptr(gu), ptr(d2), ptr(dgu), rows, f2 // 2, dtype_code(gu.dtype),
                                        stream_handle()), "ft_swiglu_bwd")
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dgu, False, w, True, rows, k, f2).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            g = w.grad
            if g is not None and g.shape == w.shape and g.is_contiguous() and g.dtype == w.dtype:
                gemm(dgu, True, x2, True, f2, k, rows, out=g, accumulate=True)
            else:
                dw = gemm(dgu, True, x2, True, f2, k, rows)
        return dx, dw


def linear_swiglu(x, w_gate_up):
    return _LinearSwiGLU.apply(x, w_gate_up)


# ---------------------------------------------------------------- attention
def _attn_impl() -> str:
    return os.environ.get("FLEXTRAIN_ATTN", "native")


def causal_attention(q, k, v, scale=None):
    """``q [B,S,H,D]``, ``k``/``v`` ``[B,S,Hkv,D]`` (views with a common row
    stride are fine) -> ``[B,S,H,D]``."""
    from . import attention
    return attention.causal_attention(q, k, v, scale)


# ------------------------------------------------- head + cross-entropy
class _LinearCrossEntropy(torch.autograd.Function):
    """Mean token cross-entropy of ``hidden @ weight.T`` without ever holding the
    full logits: rows are processed in chunks; forward keeps only the per-row
    log-sum-exp, backward recomputes each chunk's logits, turns them into
    gradients in place and feeds the two gradient GEMMs."""

    CHUNK = 4096

    @staticmethod
    def forward(ctx, hidden, weight, labels, ignore_index):
        lib = cuda_lib()
        n, h = hidden.shape
        v = weight.shape[0]
        hidden = hidden.contiguous()
        labels = labels.contiguous()
        dev = hidden.device
        lse = torch.empty(n, dtype=torch.float32, device=dev)
        loss_sum = torch.zeros(1, dtype=torch.float32, device=dev)
        count = torch.zeros(1, dtype=torch.int32, device=dev)
        _check(lib.ft_count_valid(ptr(labels), n, ignore_index, v, ptr(count), stream_handle()),
               "ft_count_valid")
        chunk = _LinearCrossEntropy.CHUNK
        logits = torch.empty(min(chunk, n), v, dtype=hidden.dtype, device=dev)
        for lo in range(0, n, chunk):
            rows = min(chunk, n - lo)
            gemm(hidden[lo:lo + rows], False, weight, False, rows, v, h, out=logits[:rows])
            _check(lib.ft_xent_fwd(ptr(logits), logits.stride(0), ptr(labels[lo:]), rows, v,
                                   ignore_index, ptr(lse[lo:]), ptr(loss_sum),
                                   dtype_code(logits.dtype), stream_handle()), "ft_xent_fwd")
        countf = count.float().clamp_(min=1.0)
        ctx.save_for_backward(hidden, weight, labels, lse, countf)
        ctx.ignore_index = ignore_index
        return (loss_sum / countf).squeeze(0)

    @staticmethod
    def backward(ctx, grad_out):
        hidden, weight, labels, lse, countf = ctx.saved_tensors
        lib = cuda_lib()
        n, h = hidden.shape
        v = weight.shape[0]
        dev = hidden.device
        chunk = _LinearCrossEntropy.CHUNK
        scale = (grad_out.float().reshape(1) / countf).contiguous()
        dh = torch.empty_like(hidden)
        wg = weight.grad
        inplace = wg is not None and wg.shape == weight.shape and wg.is_contiguous() \
            and wg.dtype == weight.dtype
        dw = wg if inplace else torch.zeros_like(weight)
        logits = torch.empty(min(chunk, n), v, dtype=hidden.dtype, device=dev)
        for lo in range(0, n, chunk):
            rows = min(chunk, n - lo)
            hc = hidden[lo:lo + rows]
            lg = logits[:rows]
            gemm(hc, False, weight, False, rows, v, h, out=lg)
            _check(lib.ft_xent_bwd(ptr(lg), lg.stride(0), ptr(labels[lo:]), rows, v, ctx.ignore_index,
                                   ptr(lse[lo:]), ptr(scale), 1.0, dtype_code(lg.dtype),
                                   stream_handle()), "ft_xent_bwd")
            gemm(lg, False, weight, True, rows, h, v, out=dh[lo:lo + rows])
            gemm(lg, True, hc, True, v, h, rows, out=dw, accumulate=True)
        return dh, (None if inplace else dw), None, None


def linear_cross_entropy(hidden, weight, labels, ignore_index=-100):
    return _LinearCrossEntropy.apply(hidden, weight, labels, int(ignore_index))
