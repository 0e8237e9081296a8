"""GPT family on one B200, the in-place parameter layout with a host optimizer share, and
the row-resident norm / bias / GELU kernels and the SwiGLU GEMM epilogue against fp32
PyTorch."""
import math
import os

import pytest
import torch
import torch.nn.functional as TF

pytestmark = pytest.mark.gpu

def _dev():
    return torch.device("cuda", 0)


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm().clamp_min(1e-12)).item()


def _run_engine(split, steps=4, tie=True):
    from flextrain_b200.models.gpt import preset
    from flextrain_b200.testing import build_gpt_engine, reset_runtime
    reset_runtime()
    dev = _dev()
    cfg = preset("tiny", num_layers=4, hidden=256, num_heads=4, vocab=1024, seq_len=256,
                 tie_embeddings=tie)
    gen = torch.Generator().manual_seed(1)
    data = [torch.randint(0, cfg.vocab, (2, cfg.seq_len + 1), generator=gen).to(dev) for _ in range(2)]
    it = {"i": 0}

    def batch_fn():
        t = data[it["i"] % 2]
        it["i"] += 1
        return t[:, :-1], t[:, 1:]

    ft_cfg = {"batch_size": 4, "micro_batch_size": 2,
              "mixed_precision": {"device_dtype": "bf16"}, "split_ratio": split}
    model, opt, eng = build_gpt_engine(cfg, ft_cfg, batch_fn, lr=1e-3, init_device=dev,
                                       dtype=torch.bfloat16)
    losses = []
    for _ in range(steps):
        r = eng.train_iteration()
        losses.append(sum(float(x) for x in r) / len(r))
    eng.synchronize()
    eng.shutdown()
    reset_runtime()
    return losses


ALL_HBM = {"parameter": [1.0, 0.0], "optimizer": [1.0, 0.0], "checkpoint": [1.0, 0.0],
           "gradient": [1.0, 0.0]}
TIERED = {"parameter": [0.5, 0.5], "optimizer": [0.25, 0.75], "checkpoint": [0.0, 1.0],
          "gradient": [0.5, 0.5], "alpha": 0.25}


def test_gpt_trains_through_the_engine():
    base = _run_engine(ALL_HBM)
    assert abs(base[0] - math.log(1024)) < 0.2
    assert base[-1] < base[0] - 0.05
    tiered = _run_engine(TIERED)
    assert max(abs(a - b) for a, b in zip(base, tiered)) < 2e-3, (base, tiered)


def test_parameters_in_place_with_host_optimizer_share():
    """The single-GPU benchmark layout on a tiny Llama: every parameter in HBM (units are
    computed straight from the base copy, nothing is gathered) while part of the optimizer
    state is updated on the host and copied back asynchronously."""
    from flextrain_b200.models.llama import preset
    from flextrain_b200.testing import build_llama_engine, reset_runtime

    def run(split, buffers):
        reset_runtime()
        dev = _dev()
        cfg = preset("tiny", num_layers=4, hidden=256, num_heads=4, ffn=768, vocab=1024, seq_len=256)
        gen = torch.Generator().manual_seed(1)
        data = [torch.randint(0, cfg.vocab, (2, cfg.seq_len + 1), generator=gen).to(dev) for _ in range(2)]
        it = {"i": 0}

        def batch_fn():
            t = data[it["i"] % 2]
            it["i"] += 1
            return t[:, :-1], t[:, 1:]

        ft_cfg = {"batch_size": 4, "micro_batch_size": 2, "mixed_precision": {"device_dtype": "bf16"},
                  "split_ratio": split, "engine": {"num_unit_buffers": buffers}}
        model, opt, eng = build_llama_engine(cfg, ft_cfg, batch_fn, lr=1e-3, init_device=dev,
                                             dtype=torch.bfloat16)
        losses = []
        for _ in range(5):
            r = eng.train_iteration()
            losses.append(sum(float(x) for x in r) / len(r))
        eng.synchronize()
        health = eng.health()
        eng.shutdown()
        reset_runtime()
        return losses, health

    base, _ = run(ALL_HBM, 2)
    split = {"parameter": [1.0, 0.0], "optimizer": [0.5, 0.5], "checkpoint": [1.0, 0.0],
             "gradient": [1.0, 0.0], "alpha": 0.25}
    got, health = run(split, 3)
    assert max(abs(a - b) for a, b in zip(base, got)) < 2e-3, (base, got)
    assert health["skipped_steps"] == 0


@pytest.mark.parametrize("rows,h", [(5, 256), (64, 1024), (33, 5120), (17, 8192), (9, 12288)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_layernorm_kernels(rows, h, dtype):
    from flextrain_b200.ops import cuda_ops
    torch.manual_seed(rows + h)
    x = torch.randn(rows, h, device=_dev(), dtype=dtype, requires_grad=True)
    w = (1 + 0.1 * torch.randn(h, device=_dev())).to(dtype).requires_grad_()
    b = (0.1 * torch.randn(h, device=_dev())).to(dtype).requires_grad_()
    dy = torch.randn(rows, h, device=_dev(), dtype=dtype)
    y = cuda_ops.layernorm(x, w, b, 1e-5)
    gx, gw, gb = torch.autograd.grad(y, (x, w, b), dy)
    xf, wf, bf = (t.detach().float().requires_grad_() for t in (x, w, b))
    yf = TF.layer_norm(xf, (h,), wf, bf, 1e-5)
    fx, fw, fb = torch.autograd.grad(yf, (xf, wf, bf), dy.float())
    assert _rel_err(y, yf) < 1e-2
    assert _rel_err(gx, fx) < 1e-2 and _rel_err(gw, fw) < 1e-2 and _rel_err(gb, fb) < 1e-2


@pytest.mark.parametrize("rows,h", [(7, 256), (130, 4096), (33, 5120), (10, 8192)])
def test_rmsnorm_row_kernels(rows, h):
    from flextrain_b200.ops import cuda_ops, reference as ref
    torch.manual_seed(rows * 3 + h)
    x = torch.randn(rows, h, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(h, device=_dev())).to(torch.bfloat16).requires_grad_()
    dy = torch.randn(rows, h, device=_dev(), dtype=torch.bfloat16)
    y = cuda_ops.rmsnorm_rows(x, w, 1e-5)
    gx, gw = torch.autograd.grad(y, (x, w), dy)
    xf, wf = (t.detach().float().requires_grad_() for t in (x, w))
    yf = ref.rmsnorm(xf, wf, 1e-5)
    fx, fw = torch.autograd.grad(yf, (xf, wf), dy.float())
    assert _rel_err(y, yf) < 1e-2 and _rel_err(gx, fx) < 1e-2 and _rel_err(gw, fw) < 1e-2


@pytest.mark.parametrize("rows,n", [(3, 8), (100, 264), (513, 1024), (64, 20480)])
@pytest.mark.parametrize("act", [0, 1])
def test_bias_activation_kernels(rows, n, act):
    from flextrain_b200.ops import cuda_ops
    torch.manual_seed(rows + n + act)
    dt = torch.bfloat16
    x = torch.randn(rows, n, device=_dev(), dtype=dt)
    b = torch.randn(n, device=_dev(), dtype=dt, requires_grad=True)
    dy = torch.randn(rows, n, device=_dev(), dtype=dt)
    xin = (x.clone() * 1.0).requires_grad_()           # non-leaf input: act 0 works in place on it
    pre = xin * 1.0
    y = cuda_ops.bias_add(pre, b) if act == 0 else cuda_ops.bias_gelu(pre, b)
    gx, gb = torch.autograd.grad(y, (xin, b), dy)
    xf, bf = x.float().requires_grad_(), b.detach().float().requires_grad_()
    yf = xf + bf if act == 0 else TF.gelu(xf + bf, approximate="tanh")
    fx, fb = torch.autograd.grad(yf, (xf, bf), dy.float())
    assert _rel_err(y, yf) < 1e-2
    assert _rel_err(gx, fx) < 1e-2 and _rel_err(gb, fb) < 2e-2


def test_gpt_engine_native_elementwise_against_aten(monkeypatch):
    native = _run_engine(ALL_HBM)
    monkeypatch.setenv("FLEXTRAIN_GPT_ELEMENTWISE", "aten")
    aten = _run_engine(ALL_HBM)
    assert max(abs(a - b) for a, b in zip(aten, native)) < 3e-2, (aten, native)
    assert native[-1] < native[0] - 0.05


@pytest.mark.parametrize("rows,k,f", [(256, 256, 128), (520, 320, 384), (4096, 1024, 2816), (200, 256, 136)])
def test_swiglu_in_the_gemm_epilogue(rows, k, f):
    """Projection GEMM with the activation in its epilogue against the two-kernel path
    (values and all gradients); the last shape is outside the fused kernel and must take
    the fallback inside the same op."""
    from flextrain_b200.ops import cuda_ops
    from flextrain_b200.ops.native import cuda_lib
    torch.manual_seed(rows + k + f)
    x = (torch.randn(rows, k, device=_dev()) * 0.5).to(torch.bfloat16).requires_grad_()
    w = (torch.randn(2 * f, k, device=_dev()) * 0.05).to(torch.bfloat16).requires_grad_()
    dy = torch.randn(rows, f, device=_dev(), dtype=torch.bfloat16)
    want = cuda_ops.swiglu(cuda_ops.linear(x, w))
    wx, ww = torch.autograd.grad(want, (x, w), dy)
    got = cuda_ops.linear_swiglu(x, w)
    gx, gw = torch.autograd.grad(got, (x, w), dy)
    torch.cuda.synchronize()
    assert cuda_lib().ft_gemm_error() == 0
    assert _rel_err(got, want) < 1e-2 and _rel_err(gx, wx) < 1e-2 and _rel_err(gw, ww) < 1e-2
    with torch.no_grad():                                  # no backward ahead: nothing but the activation is written
        assert _rel_err(cuda_ops.linear_swiglu(x, w), want) < 1e-2
