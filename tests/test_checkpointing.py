import pytest
import torch

from flextrain_b200 import checkpointing as ck


def test_recompute_matches_plain_backward_with_dropout():
    torch.manual_seed(0)
    lin = torch.nn.Linear(16, 16)
    drop = torch.nn.Dropout(0.5)

    def fn(x, scale):
        return drop(lin(x)) * scale

    x = torch.randn(4, 16)
    out, ctx = ck.checkpointed_forward(fn, x, 2.0)
    assert not out.requires_grad and ctx.fwd_args[1] == 2.0
    fired = []
    ck.set_post_recomputation_function(lambda: fired.append(1))
    torch.manual_seed(123)                       # ambient RNG moves on; recompute must replay the old state
    before = torch.get_rng_state()
    gx, gscale = ck.checkpointed_backward(ctx, torch.ones_like(out))
    assert fired == [1] and gscale is None
    assert torch.equal(before, torch.get_rng_state())     # ambient RNG restored after recompute
    mask = (out != 0).float()
    want = (mask * 2.0 / 0.5) @ lin.weight
    assert torch.allclose(gx, want, atol=1e-6)
    gx2, _ = ck.checkpointed_backward(ctx, torch.ones_like(out))
    assert fired == [1]                                    # the hook is one-shot
    assert torch.allclose(gx2, gx)


def test_detach_and_retrieve_helpers():
    a = torch.randn(3, requires_grad=True) * 2
    d = ck.detach_variable((a, 5, torch.tensor([1, 2])))
    assert d[0].requires_grad and d[0].grad_fn is None and d[1] == 5 and not d[2].requires_grad
    assert ck.detach_variable(a).requires_grad
    assert ck.detach_variable(7) == 7
    assert ck.retrieve_tensor((1, a, "x")) is a
    with pytest.raises(ValueError):
        ck.retrieve_tensor((a, a))
    d[0].sum().backward()
    assert ck.retrieve_tensor_grads(d)[0] is d[0].grad and ck.retrieve_tensor_grads(d)[1] is None


def test_rng_tracker_api():
    tr = ck.get_cuda_rng_tracker()
    ck.model_parallel_cuda_manual_seed(1234)
    assert "model-parallel-rng" in tr.get_states()
    with pytest.raises(ValueError):
        tr.add("model-parallel-rng", 99)
    with pytest.raises(ValueError):
        tr.add("other", 1234 + 2718)
    with tr.fork():
        pass
    with pytest.raises(KeyError):
        with tr.fork("missing"):
            pass
    states = tr.get_states()
    tr.reset()
    assert tr.get_states() == {}
    tr.set_states(states)
    assert "model-parallel-rng" in tr.get_states()
