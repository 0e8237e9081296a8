"""Numerics of every sm_100a kernel against a plain PyTorch fp32 statement of
the same op (small and odd shapes, canary words around outputs)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from flextrain_b200.ops import reference as ref


def _dev():
    return torch.device("cuda", 0)


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm().clamp_min(1e-12)).item()


@pytest.fixture(autouse=True)
def _gemm_error_word():
    yield
    from flextrain_b200.ops.native import cuda_lib
    torch.cuda.synchronize()
    assert cuda_lib().ft_gemm_error() == 0, "a bounded wait inside the GEMM kernel expired"


GEMM_SHAPES = [(128, 256, 64), (256, 512, 128), (384, 768, 320), (200, 264, 136), (1024, 1024, 1024),
               (4096, 1536, 512), (136, 4096, 8192)]


@pytest.mark.parametrize("m,n,k", GEMM_SHAPES)
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_gemm_layouts(m, n, k, a_mn, b_mn, dtype):
    from flextrain_b200.ops.cuda_ops import gemm
    torch.manual_seed(m * 7 + n * 3 + k)
    if dtype == torch.float16 and (m, n, k) not in GEMM_SHAPES[:4]:
        pytest.skip("fp16 covered on the small shapes")
    a = torch.randn(m, k, device=_dev(), dtype=dtype)
    b = torch.randn(n, k, device=_dev(), dtype=dtype)
    a_st = a.t().contiguous() if a_mn else a
    b_st = b.t().contiguous() if b_mn else b
    # canary rows around the output
    pad = torch.full((m + 2, n), 7.0, device=_dev(), dtype=dtype)
    out = pad[1:-1]
    gemm(a_st, a_mn, b_st, b_mn, m, n, k, out=out)
    want = a.float() @ b.float().t()
    assert _rel_err(out, want) < 1e-2
    assert torch.all(pad[0] == 7.0) and torch.all(pad[-1] == 7.0)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_accumulate_and_fp32_out(out_dtype):
    from flextrain_b200.ops.cuda_ops import gemm
    m, n, k = 256, 512, 192
    a = torch.randn(m, k, device=_dev(), dtype=torch.bfloat16)
    b = torch.randn(n, k, device=_dev(), dtype=torch.bfloat16)
    c0 = torch.randn(m, n, device=_dev(), dtype=out_dtype)
    c = c0.clone()
    gemm(a, False, b, False, m, n, k, out=c, accumulate=True)
    want = c0.float() + a.float() @ b.float().t()
    assert _rel_err(c, want) < (1e-2 if out_dtype == torch.bfloat16 else 1e-5 * 50)
    c2 = torch.empty(m, n, device=_dev(), dtype=out_dtype)
    gemm(a, False, b, False, m, n, k, out=c2)
    assert _rel_err(c2, a.float() @ b.float().t()) < (1e-2 if out_dtype == torch.bfloat16 else 1e-4)


def test_linear_autograd_matches_reference():
    from flextrain_b200.ops.cuda_ops import linear
    x = torch.randn(2, 96, 320, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    w = torch.randn(520, 320, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    dy = torch.randn(2, 96, 520, device=_dev(), dtype=torch.bfloat16)
    y = linear(x, w)
    y.backward(dy)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = torch.nn.functional.linear(xr, wr)
    yr.backward(dy.float())
    assert _rel_err(y, yr) < 1e-2
    assert _rel_err(x.grad, xr.grad) < 1e-2
    assert _rel_err(w.grad, wr.grad) < 1e-2


@pytest.mark.parametrize("rows,k,n", [(192, 320, 520), (40, 128, 256), (300, 512, 1024)])
def test_linear_add_puts_the_residual_in_the_epilogue(rows, k, n):
    """``res + x w^T`` from one GEMM launch (CTA-pair kernel above 128 rows, single-CTA below),
    against fp32 PyTorch, with all three gradients; the residual itself must stay untouched."""
    from flextrain_b200.ops.cuda_ops import linear_add
    x = torch.randn(rows, k, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(n, k, device=_dev()) / k ** 0.5).to(torch.bfloat16).requires_grad_()
    res = torch.randn(rows, n, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    keep = res.detach().clone()
    dy = torch.randn(rows, n, device=_dev(), dtype=torch.bfloat16)
    y = linear_add(x, w, res)
    y.backward(dy)
    assert torch.equal(res.detach(), keep)
    xr, wr, rr = (t.detach().float().requires_grad_() for t in (x, w, res))
    yr = rr + torch.nn.functional.linear(xr, wr)
    yr.backward(dy.float())
    assert _rel_err(y, yr) < 1e-2
    assert _rel_err(x.grad, xr.grad) < 1e-2 and _rel_err(w.grad, wr.grad) < 1e-2
    assert torch.equal(res.grad, dy)


def test_linear_accumulates_into_existing_grad():
    from flextrain_b200.ops.cuda_ops import linear
    x = torch.randn(256, 128, device=_dev(), dtype=torch.bfloat16)
    w = torch.randn(256, 128, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    w.grad = torch.ones_like(w)
    linear(x, w).sum().backward()
    want = 1.0 + x.float().sum(0)[None, :].expand(256, 128)
    assert _rel_err(w.grad, want) < 1e-2


@pytest.mark.parametrize("rows,h", [(1, 256), (37, 1024), (300, 4096), (16, 8192)])
def test_rmsnorm(rows, h):
    from flextrain_b200.ops.cuda_ops import rmsnorm
    x = torch.randn(rows, h, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(h, device=_dev())).to(torch.bfloat16).requires_grad_()
    dy = torch.randn(rows, h, device=_dev(), dtype=torch.bfloat16)
    y = rmsnorm(x, w, 1e-5)
    y.backward(dy)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = ref.rmsnorm(xr, wr, 1e-5)
    yr.backward(dy.float())
    assert _rel_err(y, yr) < 1e-2
    assert _rel_err(x.grad, xr.grad) < 1e-2
    assert _rel_err(w.grad, wr.grad) < 2e-2


@pytest.mark.parametrize("rows,h", [(3, 256), (64, 4096), (33, 5120), (17, 8192)])
def test_add_rmsnorm_fuses_the_residual_both_ways(rows, h):
    """``s = x + r`` and ``rmsnorm(s)`` in one kernel, and in the backward the gradient that
    reaches ``s`` directly added to the one through the norm: against fp32 PyTorch."""
    from flextrain_b200.ops.functional import add_rmsnorm
    dev = _dev()
    x = torch.randn(rows, h, device=dev, dtype=torch.bfloat16, requires_grad=True)
    r = torch.randn(rows, h, device=dev, dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(h, device=dev)).to(torch.bfloat16).requires_grad_()
    ds = torch.randn(rows, h, device=dev, dtype=torch.bfloat16)
    dy = torch.randn(rows, h, device=dev, dtype=torch.bfloat16)
    s, y = add_rmsnorm(x, r, w, 1e-5)
    torch.autograd.backward([s, y], [ds, dy])
    xr, rr, wr = (t.detach().float().requires_grad_() for t in (x, r, w))
    sr = (xr + rr).to(torch.bfloat16).float()          # the stored sum is rounded to bf16
    sr2 = xr + rr
    yr = ref.rmsnorm(sr2, wr, 1e-5)
    torch.autograd.backward([sr2, yr], [ds.float(), dy.float()])
    assert torch.equal(s.float(), sr)
    assert _rel_err(y, yr) < 1e-2
    assert _rel_err(x.grad, xr.grad) < 1e-2
    assert _rel_err(r.grad, rr.grad) < 1e-2
    assert _rel_err(w.grad, wr.grad) < 2e-2


@pytest.mark.parametrize("d", [64, 128])
def test_rope_and_inplace_heads(d):
    from flextrain_b200.ops.cuda_ops import rope, rope_heads_inplace
    B, S, H = 2, 48, 6
    cos, sin = ref.rope_tables(S, d, 10000.0, device=_dev())
    x = torch.randn(B, S, H, d, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    dy = torch.randn_like(x)
    y = rope(x, cos, sin)
    y.backward(dy)
    xr = x.detach().float().requires_grad_()
    yr = ref.rope(xr, cos, sin)
    yr.backward(dy.float())
    assert _rel_err(y, yr) < 1e-2 and _rel_err(x.grad, xr.grad) < 1e-2
    # fused-QKV style: rotate the first 4 of 6 heads in place, leave the rest
    packed = torch.randn(B, S, H * d, device=_dev(), dtype=torch.bfloat16)
    want = packed.clone().view(B, S, H, d)
    want[:, :, :4] = ref.rope(want[:, :, :4].float(), cos, sin).to(torch.bfloat16)
    leaf = packed.clone().requires_grad_()
    out = rope_heads_inplace(leaf * 1.0, cos, sin, 4, d)
    assert _rel_err(out, want.view(B, S, H * d)) < 1e-2
    out.backward(torch.ones_like(out))
    gr = torch.ones(B, S, H, d, device=_dev())
    gr_ref = gr.clone().requires_grad_()
    tmp = torch.cat([ref.rope(gr_ref[:, :, :4], cos, sin), gr_ref[:, :, 4:]], dim=2)
    tmp.backward(torch.ones_like(tmp))
    assert _rel_err(leaf.grad.view(B, S, H, d), gr_ref.grad) < 1e-2


def test_swiglu():
    from flextrain_b200.ops.cuda_ops import swiglu
    gu = torch.randn(70, 2 * 344, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    d = torch.randn(70, 344, device=_dev(), dtype=torch.bfloat16)
    y = swiglu(gu)
    y.backward(d)
    gr = gu.detach().float().requires_grad_()
    yr = ref.swiglu(gr)
    yr.backward(d.float())
    assert _rel_err(y, yr) < 1e-2 and _rel_err(gu.grad, gr.grad) < 1e-2


@pytest.mark.parametrize("n,h,v", [(100, 256, 1000), (5000, 128, 1024), (64, 512, 32000)])
def test_linear_cross_entropy(n, h, v):
    from flextrain_b200.ops.cuda_ops import linear_cross_entropy
    hid = (0.5 * torch.randn(n, h, device=_dev())).to(torch.bfloat16).requires_grad_()
    w = (0.05 * torch.randn(v, h, device=_dev())).to(torch.bfloat16).requires_grad_()
    labels = torch.randint(0, v, (n,), device=_dev())
    labels[::7] = -100
    loss = linear_cross_entropy(hid, w, labels)
    (loss * 3.0).backward()
    hr, wr = hid.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    lr = ref.linear_cross_entropy(hr, wr, labels)
    (lr * 3.0).backward()
    assert abs(loss.item() - lr.item()) < 2e-2
    assert _rel_err(hid.grad, hr.grad) < 3e-2
    assert _rel_err(w.grad, wr.grad) < 3e-2


@pytest.mark.parametrize("gdt", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("n", [1, 1000, 65536 + 13])
def test_adam_cuda_matches_host_kernel(gdt, n):
    from flextrain_b200.ops.adam.cpu_adam import cpu_adam_update
    from flextrain_b200.ops.adam.gpu_adam import device_adam_update

    class Owner:
        defaults = dict(lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, bias_correction=True)
        adamw_mode = True

    torch.manual_seed(n)
    p = torch.randn(n)
    g = (torch.randn(n) * 64).to(gdt)
    m, v = torch.rand(n) * 0.1, torch.rand(n) * 0.1
    pd, gd, md, vd = (t.to(_dev()) for t in (p, g, m, v))
    out = torch.empty(n, device=_dev(), dtype=torch.bfloat16)
    outc = torch.empty(n, dtype=torch.bfloat16)
    flag = torch.zeros(1, dtype=torch.int32, device=_dev())
    for step in (1, 2, 3):
        device_adam_update({}, step, Owner, pd, gd, [md, vd], out, grad_scale=1 / 64, skip_flag=flag)
        cpu_adam_update(step, 1e-3, 0.9, 0.999, 1e-8, 0.01, True, True, p, g, m, v, outc,
                        grad_scale=1 / 64)
    assert torch.allclose(pd.cpu(), p, rtol=1e-5, atol=1e-6)
    assert torch.allclose(md.cpu(), m, rtol=1e-5, atol=1e-7)
    assert torch.allclose(vd.cpu(), v, rtol=1e-5, atol=1e-7)
    assert torch.allclose(out.cpu().float(), outc.float(), rtol=1e-2, atol=1e-3)
    # a raised skip flag leaves everything untouched
    flag.fill_(1)
    before = pd.clone()
    device_adam_update({}, 4, Owner, pd, gd, [md, vd], out, skip_flag=flag)
    assert torch.equal(before, pd)


def test_finite_flag_and_accumulate():
    from flextrain_b200.ops.adam.gpu_adam import has_nonfinite
    from flextrain_b200.ops.elementwise import accumulate_and_zero, cast_copy
    x = torch.randn(100003, device=_dev(), dtype=torch.bfloat16)
    assert not has_nonfinite(x)
    x[77777] = float("inf")
    assert has_nonfinite(x)
    x[77777] = float("nan")
    assert has_nonfinite(x)
    acc = torch.randn(4096 * 3 + 5, device=_dev())
    src = torch.randn(4096 * 3 + 5, device=_dev()).to(torch.bfloat16)
    want = acc + src.float()
    accumulate_and_zero(acc, src)
    assert torch.allclose(acc, want) and torch.all(src == 0)
    acc8 = torch.randn(8192, device=_dev())
    src8 = torch.randn(8192, device=_dev()).to(torch.bfloat16)
    want8 = acc8 + src8.float()
    accumulate_and_zero(acc8, src8)
    assert torch.allclose(acc8, want8) and torch.all(src8 == 0)
    dst = torch.empty(1001, device=_dev(), dtype=torch.bfloat16)
    srcf = torch.randn(1001, device=_dev())
    cast_copy(dst, srcf)
    assert torch.equal(dst, srcf.to(torch.bfloat16))


@pytest.mark.parametrize("S", [320, 1000])     # 1000: the last block's valid rows end inside a warp
@pytest.mark.parametrize("hq,hkv,d,dt", [(4, 4, 64, torch.bfloat16), (8, 2, 128, torch.bfloat16),
                                         (4, 2, 128, torch.float16)])
def test_causal_attention(hq, hkv, d, dt, S):
    from flextrain_b200.ops.functional import causal_attention
    B = 2
    q = torch.randn(B, S, hq, d, device=_dev(), dtype=dt, requires_grad=True)
    k = torch.randn(B, S, hkv, d, device=_dev(), dtype=dt, requires_grad=True)
    v = torch.randn(B, S, hkv, d, device=_dev(), dtype=dt, requires_grad=True)
    do = torch.randn(B, S, hq, d, device=_dev(), dtype=dt)
    o = causal_attention(q, k, v)
    o.backward(do)
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    orf = ref.causal_attention(qr, kr, vr)
    orf.backward(do.float())
    assert _rel_err(o, orf) < 2e-2
    assert _rel_err(q.grad, qr.grad) < 3e-2
    assert _rel_err(k.grad, kr.grad) < 3e-2
    assert _rel_err(v.grad, vr.grad) < 3e-2


def _attention_oracle(q, k, v, scale):
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(Hq // Hkv, 1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(Hq // Hkv, 1)
    s = qf @ kf.transpose(-1, -2) * scale
    mask = torch.ones(S, S, device=q.device, dtype=torch.bool).tril()
    s = s.masked_fill(~mask, float("-inf"))
    return (torch.softmax(s, -1) @ vf).permute(0, 2, 1, 3), torch.logsumexp(s, -1)


@pytest.mark.parametrize("shape", [
    (1, 128, 1, 1, 128, torch.bfloat16, 1.0),      # one block, second tile of the pair absent
    (1, 256, 1, 1, 128, torch.bfloat16, 1.0),      # exactly one pair
    (2, 320, 4, 4, 64, torch.bfloat16, 1.0),       # odd number of blocks, head dim 64
    (2, 384, 8, 2, 128, torch.bfloat16, 1.0),      # grouped-query
    (1, 1024, 4, 1, 128, torch.float16, 1.0),
    (1, 1000, 2, 2, 128, torch.bfloat16, 1.0),     # sequence not a multiple of the block
    (1, 2048, 2, 1, 128, torch.bfloat16, 6.0),     # large scores: the running maximum keeps growing
])
def test_attention_forward(shape):
    """The forward kernel against the fp32 oracle: output and log-sum-exp, including
    shapes that exercise the absent second tile, the ragged last block and the lazy
    rescale of the accumulator."""
    import math
    from flextrain_b200.ops.attention_native import attention_forward
    from flextrain_b200.ops.native import cuda_lib
    B, S, Hq, Hkv, D, dt, amp = shape
    lib = cuda_lib()
    torch.manual_seed(S + D)
    q = (torch.randn(B, S, Hq, D, device=_dev()) * amp).to(dt)
    k = torch.randn(B, S, Hkv, D, device=_dev()).to(dt)
    v = torch.randn(B, S, Hkv, D, device=_dev()).to(dt)
    scale = 1.0 / math.sqrt(D)
    for _ in range(3):                          # repeated: ordering bugs are timing dependent
        o, lse, _ = attention_forward(q, k, v, scale)
        torch.cuda.synchronize()
        assert lib.ft_gemm_error() == 0
        want_o, want_lse = _attention_oracle(q, k, v, scale)
        assert _rel_err(o, want_o) < 2e-2
        assert float((lse - want_lse).abs().max()) < 2e-2


def test_attention_timeline_instantiations_compute_the_same_and_fill_the_trace():
    """The timeline builds of the two attention kernels (``benchmarks/attn_timeline.py``) must give
    the results of the regular builds, and the clocks they record must be in program order."""
    import math
    from flextrain_b200.ops.attention_backward import attention_backward
    from flextrain_b200.ops.attention_native import attention_forward
    B, S, H, D = 1, 1024, 2, 128
    torch.manual_seed(3)
    q, k, v, do = (torch.randn(B, S, H, D, device=_dev()).to(torch.bfloat16) for _ in range(4))
    scale = 1.0 / math.sqrt(D)
    o, lse, _ = attention_forward(q, k, v, scale)
    fbuf = torch.zeros(3 * 8 * 8, dtype=torch.int64, device=_dev())
    o2, lse2, _ = attention_forward(q, k, v, scale, trace=(fbuf, 0, 0))     # CTA 0: 8 K/V blocks
    torch.cuda.synchronize()
    assert torch.equal(o, o2) and torch.equal(lse, lse2)
    f = fbuf.cpu().view(3, 8, 8)
    assert (f[0, :4, :7] > 0).all() and (f[0, 4:7, :8] > 0).all() and (f[1, :6, :7] > 0).all()
    assert (f[0, 1:4, :7] >= f[0, 0:3, :7]).all()         # the product warp's sites follow one another
    assert (f[1, 1:6, :7] >= f[1, 0:5, :7]).all()         # so do the softmax warp's
    want = attention_backward(q, k, v, o, lse, do, scale)
    bbuf = torch.zeros(5 * 16 * 8, dtype=torch.int64, device=_dev())
    got = attention_backward(q, k, v, o, lse, do, scale, trace=(bbuf, 0, 0))  # CTA 0: kv block 0, 8 q blocks
    torch.cuda.synchronize()
    for a, b_ in zip(got, want):
        assert _rel_err(a, b_) < 1e-3                     # dq is summed by reduce-adds: order may differ
    t = bbuf.cpu().view(5, 16, 8)
    assert (t[1, :8] > 0).all() and (t[1, 1:8] >= t[1, 0:7]).all()
    assert (t[4, :3] > 0).all() and (t[4, 1:3] >= t[4, 0:2]).all()


def test_tensor_pipe_probe_reads_the_full_rate_for_bare_products():
    """``ft_mma_probe`` (benchmarks/mma_rate.py): back-to-back 128x128x128 products with nothing
    between them take the pipe's 512 clocks, whether A comes from shared or from tensor memory,
    and a 128x256x128 product takes 1024."""
    import ctypes
    from flextrain_b200.ops.native import cuda_lib, ptr, stream_handle
    lib = cuda_lib()
    lib.ft_mma_probe.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    lib.ft_mma_probe.restype = ctypes.c_int
    sms = torch.cuda.get_device_properties(_dev()).multi_processor_count
    out = torch.zeros(sms + 1, dtype=torch.int64, device=_dev())
    for mode, ideal in ((0, 512.0), (3, 512.0), (4, 1024.0), (6, 512.0)):
        for _ in range(2):
            out.zero_()
            assert lib.ft_mma_probe(mode, 500, ptr(out), stream_handle()) == 0
            torch.cuda.synchronize()
        per = (out[:sms].float() / 500).median().item()
        if mode == 6:                                   # with a wait, a fence and a commit per product
            assert ideal <= per < 2.0 * ideal, (mode, per)
        else:
            assert 0.98 * ideal <= per < 1.15 * ideal, (mode, per)
    assert lib.ft_gemm_error() == 0
