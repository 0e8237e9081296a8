"""LR schedule arithmetic, and the engine honouring a rate that changes every step."""
import math

import pytest
import torch

from flextrain_b200.lr_schedule import LRSchedule


class _Opt:
    def __init__(self, lrs):
        self.param_groups = [{"lr": lr} for lr in lrs]


def test_warmup_then_cosine_and_resume():
    opt = _Opt([1.0, 0.5])
    s = LRSchedule(opt, warmup_steps=4, total_steps=14, decay="cosine", min_lr_ratio=0.1)
    seen = []
    for _ in range(16):
        seen.append(opt.param_groups[0]["lr"])
        s.step()
    assert seen[:4] == [0.25, 0.5, 0.75, 1.0]
    assert abs(seen[4] - 1.0) < 1e-12 and abs(seen[9] - (0.1 + 0.9 * 0.5)) < 1e-12
    assert abs(seen[14] - 0.1) < 1e-12 and abs(seen[15] - 0.1) < 1e-12       # floor after the end
    assert all(a >= b for a, b in zip(seen[4:], seen[5:]))
    assert abs(opt.param_groups[1]["lr"] - 0.05) < 1e-12                   # own base rate
    other = _Opt([1.0, 0.5])
    r = LRSchedule(other, warmup_steps=4, total_steps=14)
    r.load_state_dict({"steps_done": 9})
    assert abs(other.param_groups[0]["lr"] - seen[9]) < 1e-12
    lin = LRSchedule(_Opt([2.0]), peak_lr=1.0, warmup_steps=0, total_steps=10, decay="linear", min_lr_ratio=0.0)
    assert abs(lin.factor(5) - 0.5) < 1e-12 and lin.current_lrs == [1.0]
    with pytest.raises(ValueError):
        LRSchedule(_Opt([1.0]), warmup_steps=5, total_steps=5)
    with pytest.raises(ValueError):
        LRSchedule(_Opt([1.0]), decay="exp", total_steps=10)


def test_engine_applies_the_rate_of_each_step(fresh_runtime):
    from flextrain_b200.models.llama import LlamaModel, preset
    from flextrain_b200.testing import build_llama_engine
    cfg = preset("tiny", num_layers=2, hidden=64, num_heads=2, ffn=136, vocab=128, seq_len=16)
    gen = torch.Generator().manual_seed(2)
    data = [torch.randint(0, 128, (2, 17), generator=gen) for _ in range(6)]
    it = {"i": 0}

    def batch_fn():
        t = data[it["i"]]
        it["i"] += 1
        return t[:, :-1], t[:, 1:]

    ft_cfg = {"batch_size": 2, "micro_batch_size": 2, "mixed_precision": {"device_dtype": "fp32"},
              "split_ratio": {"parameter": [0.5, 0.5], "optimizer": [0.5, 0.5],
                              "checkpoint": [1.0, 0.0], "gradient": [1.0, 0.0]}}
    model, opt, eng = build_llama_engine(cfg, ft_cfg, batch_fn, lr=1e-2, weight_decay=0.0, backend="gloo")
    sched = LRSchedule(opt, warmup_steps=2, total_steps=6, decay="linear", min_lr_ratio=0.0)
    eng.register_post_step_function(sched.step)
    got = [float(eng.train_iteration()[0].detach()) for _ in range(6)]
    eng.shutdown()

    torch.manual_seed(0)
    plain = LlamaModel(cfg)
    topt = torch.optim.AdamW(plain.parameters(), lr=1e-2, weight_decay=0.0)
    ref = LRSchedule(topt, warmup_steps=2, total_steps=6, decay="linear", min_lr_ratio=0.0)
    want = []
    for t in data:
        topt.zero_grad()
        loss = plain(t[:, :-1], t[:, 1:])
        loss.backward()
        topt.step()
        ref.step()
        want.append(float(loss.detach()))
    assert max(abs(a - b) for a, b in zip(got, want)) < 2e-5, (got, want)
    assert not math.isclose(want[-1], want[0])
