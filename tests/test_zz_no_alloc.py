"""The allocation-free RMSNorm backward (``ft_rmsnorm_bwd_noalloc``).

Some users of the library must not allocate device memory where they call this
op - their pools are frozen for a planned region, or the application owns the
GPU heap - so the library offers a variant whose scratch is a fixed array inside
the library.  This test drives that variant through its exported C symbol, twice
in a row (the scratch array is shared and keeps the previous call's contents),
and checks both results against the regular entry point, which takes
caller-provided scratch.  The file sorts last so a run that stops at the first
failure has already exercised everything else.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from flextrain_b200.ops.native import cuda_lib
    lib = cuda_lib()
    lib.ft_rmsnorm_bwd_noalloc.restype = ctypes.c_int
    lib.ft_rmsnorm_bwd_noalloc.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int64, ctypes.c_int,
                                                                   ctypes.c_int, ctypes.c_void_p]
    return lib


def _case(rows, h, seed, dtype=torch.bfloat16):
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(seed)
    x = torch.randn(rows, h, device=dev, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(h, device=dev, generator=g)).to(dtype)
    dy = torch.randn(rows, h, device=dev, generator=g).to(dtype)
    inv = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5).contiguous()
    return x, w, dy, inv


def _code(t):
    return 1 if t.dtype == torch.bfloat16 else 2       # dtype codes of the C entry points


def _regular(lib, x, w, dy, inv):
    rows, h = x.shape
    dx, dw = torch.empty_like(x), torch.empty_like(w)
    part = torch.empty(lib.ft_rmsnorm_bwd_parts() * h, dtype=torch.float32, device=x.device)
    rc = lib.ft_rmsnorm_bwd(x.data_ptr(), w.data_ptr(), dy.data_ptr(), inv.data_ptr(), dx.data_ptr(),
                            dw.data_ptr(), part.data_ptr(), rows, h, _code(x),
                            torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    return dx, dw


def _noalloc(lib, x, w, dy, inv):
    rows, h = x.shape
    dx, dw = torch.empty_like(x), torch.empty_like(w)      # outputs are the caller's to provide
    rc = lib.ft_rmsnorm_bwd_noalloc(x.data_ptr(), w.data_ptr(), dy.data_ptr(), inv.data_ptr(),
                                    dx.data_ptr(), dw.data_ptr(), rows, h, _code(x),
                                    torch.cuda.current_stream().cuda_stream)
    assert rc == 0, f"ft_rmsnorm_bwd_noalloc returned {rc}"
    return dx, dw


def _close(a, b, tol):
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm().clamp_min(1e-12)).item() < tol


def test_two_calls_in_a_row_match_the_regular_entry_point():
    lib = _lib()
    # second call: different shape and data, so stale scratch from the first would show
    for rows, h, seed in ((300, 4096, 1), (77, 1024, 2)):
        x, w, dy, inv = _case(rows, h, seed)
        want_dx, want_dw = _regular(lib, x, w, dy, inv)
        got_dx, got_dw = _noalloc(lib, x, w, dy, inv)
        torch.cuda.synchronize()
        assert _close(got_dx, want_dx, 1e-2)
        assert _close(got_dw, want_dw, 2e-2)


def test_rejects_sizes_beyond_the_built_in_scratch():
    lib = _lib()
    x, w, dy, inv = _case(4, 8192 + 8, 3)
    dx, dw = torch.empty_like(x), torch.empty_like(w)
    rc = lib.ft_rmsnorm_bwd_noalloc(x.data_ptr(), w.data_ptr(), dy.data_ptr(), inv.data_ptr(),
                                    dx.data_ptr(), dw.data_ptr(), 4, 8192 + 8, 1,
                                    torch.cuda.current_stream().cuda_stream)
    assert rc == -3


def test_edge_shapes_and_fp16_against_fp32_pytorch():
    """The largest hidden size the scratch covers, a single row (fewer rows than partial-sum
    slots), fp16, and an independent check: the gradients against plain fp32 PyTorch autograd
    of the same norm, not only against the other entry point."""
    from flextrain_b200.ops import reference as ref
    lib = _lib()
    for rows, h, dtype in ((5, 8192, torch.bfloat16), (1, 2048, torch.bfloat16), (40, 4096, torch.float16)):
        x, w, dy, inv = _case(rows, h, rows + h, dtype)
        got_dx, got_dw = _noalloc(lib, x, w, dy, inv)
        want_dx, want_dw = _regular(lib, x, w, dy, inv)
        torch.cuda.synchronize()
        assert _close(got_dx, want_dx, 1e-2) and _close(got_dw, want_dw, 2e-2)
        xr, wr = x.float().requires_grad_(), w.float().requires_grad_()
        ref.rmsnorm(xr, wr, 1e-5).backward(dy.float())
        assert _close(got_dx, xr.grad, 1e-2)
        assert _close(got_dw, wr.grad, 2e-2)


def test_rejects_a_hidden_size_that_is_not_a_multiple_of_eight():
    lib = _lib()
    x, w, dy, inv = _case(4, 1028, 5)
    dx, dw = torch.empty_like(x), torch.empty_like(w)
    rc = lib.ft_rmsnorm_bwd_noalloc(x.data_ptr(), w.data_ptr(), dy.data_ptr(), inv.data_ptr(),
                                    dx.data_ptr(), dw.data_ptr(), 4, 1028, 1,
                                    torch.cuda.current_stream().cuda_stream)
    assert rc == -2
