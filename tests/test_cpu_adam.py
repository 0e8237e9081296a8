import pytest
import torch

from flextrain_b200.ops.adam.cpu_adam import FlexTrainCPUAdam, cpu_adam_update
from flextrain_b200.ops.native import host_lib, ptr
from flextrain_b200.param_group import StepContext


@pytest.mark.parametrize("n", [1, 15, 16, 17, 1000, 65536 + 3, 200_003])
@pytest.mark.parametrize("adamw,wd", [(True, 0.1), (False, 0.1), (True, 0.0)])
def test_matches_torch_optimizers(n, adamw, wd):
    torch.manual_seed(n)
    p = torch.randn(n)
    ref = torch.nn.Parameter(p.clone())
    opt = (torch.optim.AdamW if adamw else torch.optim.Adam)([ref], lr=1e-3, weight_decay=wd)
    m, v = torch.zeros(n), torch.zeros(n)
    for step in range(1, 5):
        g = torch.randn(n) * 0.01
        ref.grad = g.clone()
        opt.step()
        cpu_adam_update(step, 1e-3, 0.9, 0.999, 1e-8, wd, adamw, True, p, g, m, v)
    assert torch.allclose(p, ref.data, rtol=1e-5, atol=1e-6)
    assert torch.allclose(m, opt.state[ref]["exp_avg"], rtol=1e-4, atol=1e-8)
    assert torch.allclose(v, opt.state[ref]["exp_avg_sq"], rtol=1e-4, atol=1e-10)


@pytest.mark.parametrize("gdt", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("odt", [torch.bfloat16, torch.float16, torch.float32])
def test_simd_path_equals_scalar_path_and_copies(gdt, odt):
    n = 70_001
    torch.manual_seed(1)
    p0, g = torch.randn(n), (torch.randn(n) * 128).to(gdt)
    outs = []
    for scalar in (False, True):
        p, m, v = p0.clone(), torch.zeros(n), torch.zeros(n)
        out = torch.empty(n, dtype=odt)
        bad = cpu_adam_update(3, 1e-3, 0.9, 0.95, 1e-8, 0.01, True, True, p, g, m, v, out,
                              grad_scale=1 / 128, force_scalar=scalar)
        assert not bad
        outs.append((p, m, v, out))
    for a, b in zip(*outs):
        assert torch.equal(a, b)
    assert torch.equal(outs[0][3], outs[0][0].to(odt))      # bf16 copy is a true bf16 rounding


def test_reports_nonfinite_gradients_and_thread_count_invariance():
    n = 300_000
    g = torch.randn(n)
    res = []
    for threads in (1, 4):
        p, m, v = torch.ones(n), torch.zeros(n), torch.zeros(n)
        cpu_adam_update(1, 1e-3, 0.9, 0.999, 1e-8, 0.0, True, True, p, g, m, v, threads=threads)
        res.append(p)
    assert torch.equal(res[0], res[1])
    g[12345] = float("nan")
    p, m, v = torch.ones(n), torch.zeros(n), torch.zeros(n)
    assert cpu_adam_update(1, 1e-3, 0.9, 0.999, 1e-8, 0.0, True, True, p, g, m, v)
    assert host_lib().ft_has_nonfinite(ptr(g), 0, n, 0) == 1


def test_optimizer_object_steps_contexts_and_profiles():
    opt = FlexTrainCPUAdam(lr=1e-2, weight_decay=0.0)
    n = 1000
    states = opt._init_optimizer_states(n, torch.float32)
    assert len(states) == opt.optimizer_state_per_element == 2
    master, grad = torch.ones(n), torch.ones(n)
    half = torch.empty(n, dtype=torch.bfloat16)
    ctx = StepContext({"lr": 1e-2, "step": 1}, master, grad, states, half)
    assert not opt.step(ctx)
    assert torch.allclose(master, torch.full((n,), 0.99), atol=1e-6)
    assert torch.equal(half, master.to(torch.bfloat16))
    assert opt.profile_step(4096, torch.bfloat16, torch.float32) > 0
    assert host_lib().ft_adam_simd_level() in (0, 512)


def test_host_casts_and_memcpy():
    lib = host_lib()
    x = torch.randn(100_001)
    b = torch.empty(100_001, dtype=torch.bfloat16)
    lib.ft_cast_from_f32(ptr(x), ptr(b), 1, x.numel(), 2)
    assert torch.equal(b, x.to(torch.bfloat16))
    back = torch.empty_like(x)
    lib.ft_cast_to_f32(ptr(b), 1, ptr(back), x.numel(), 2)
    assert torch.equal(back, b.float())
    dst = torch.empty_like(x)
    lib.ft_host_memcpy(ptr(dst), ptr(x), x.numel() * 4, 3)
    assert torch.equal(dst, x)
