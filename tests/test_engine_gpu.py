"""Engine on one B200: bf16 tiny Llama through the sm_100a kernels; every tier
layout must give the same training trajectory as the all-HBM layout, that
trajectory must follow an fp32 PyTorch model trained with AdamW, and an overflow
in the last unit to finish must reach the step's verdict."""
import tempfile

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(split, steps=4, mbpr=2, interval=1, buffers=2, swap_dir=None, dtype="bf16"):
    from flextrain_b200.models.llama import preset
    from flextrain_b200.testing import build_llama_engine, reset_runtime
    reset_runtime()
    dev = torch.device("cuda", 0)
    cfg = preset("tiny", num_layers=4, hidden=256, num_heads=4, ffn=768, vocab=1024, seq_len=256)
    gen = torch.Generator().manual_seed(1)
    data = [torch.randint(0, cfg.vocab, (2, cfg.seq_len + 1), generator=gen).to(dev)
            for _ in range(mbpr)]
    it = {"i": 0}

    def batch_fn():
        t = data[it["i"] % mbpr]
        it["i"] += 1
        return t[:, :-1], t[:, 1:]

    ft_cfg = {"batch_size": 2 * mbpr, "micro_batch_size": 2, "checkpoint_interval": interval,
              "mixed_precision": {"device_dtype": dtype, "dynamic_loss_scaling": dtype == "fp16",
                                  "initial_scale_power": 10},
              "split_ratio": split, "engine": {"num_unit_buffers": buffers}}
    if swap_dir:
        ft_cfg["nvme_swap"] = {"swap_dir": swap_dir}
    model, opt, eng = build_llama_engine(cfg, ft_cfg, batch_fn, lr=1e-3, init_device=dev,
                                         dtype=torch.bfloat16 if dtype == "bf16" else torch.float16)
    losses = []
    for _ in range(steps):
        r = eng.train_iteration()
        losses.append(sum(float(x) for x in r) / len(r))
    eng.synchronize()
    health = eng.health()
    eng.shutdown()
    reset_runtime()
    return losses, health


ALL_HBM = {"parameter": [1.0, 0.0], "optimizer": [1.0, 0.0], "checkpoint": [1.0, 0.0],
           "gradient": [1.0, 0.0]}


def test_loss_goes_down_and_starts_near_log_vocab():
    import math
    losses, health = _run(ALL_HBM, steps=6)
    assert abs(losses[0] - math.log(1024)) < 0.2
    assert losses[-1] < losses[0] - 0.05
    assert health["skipped_steps"] == 0


@pytest.mark.parametrize("split", [
    {"parameter": [0.0, 1.0], "optimizer": [0.0, 1.0], "checkpoint": [0.0, 1.0], "gradient": [0.0, 1.0]},
    {"parameter": [0.5, 0.5], "optimizer": [0.25, 0.75], "checkpoint": [0.5, 0.5], "gradient": [0.5, 0.5],
     "alpha": 0.5},
    {"parameter": [0.25, 0.75], "optimizer": [0.6, 0.4], "checkpoint": [1.0, 0.0], "gradient": [1.0, 0.0]},
])
def test_tier_layouts_agree_with_all_hbm(split):
    base, _ = _run(ALL_HBM)
    got, _ = _run(split, buffers=3)
    assert max(abs(a - b) for a, b in zip(base, got)) < 2e-3, (base, got)


def test_nvme_tiers_and_interval2():
    base, _ = _run(ALL_HBM, interval=2)
    with tempfile.TemporaryDirectory() as d:
        split = {"parameter": [0.25, 0.25], "optimizer": [0.25, 0.25], "checkpoint": [0.25, 0.25],
                 "gradient": [0.5, 0.5], "alpha": 0.2}
        got, _ = _run(split, interval=2, swap_dir=d)
    assert max(abs(a - b) for a, b in zip(base, got)) < 2e-3, (base, got)


def test_fp16_dynamic_loss_scale_runs():
    losses, health = _run(ALL_HBM, steps=5, dtype="fp16")
    assert all(l == l for l in losses)
    assert losses[-1] < losses[0]


def test_bf16_engine_follows_an_fp32_pytorch_adamw_trajectory():
    """Five steps of the bf16 engine (native kernels, tiered state) against a plain fp32
    PyTorch model of the same weights trained with ``torch.optim.AdamW`` on the same data:
    a systematic error shared by every tier layout (a wrong gradient scale, a wrong
    update rule) cannot hide behind the layouts agreeing with each other."""
    from flextrain_b200.models.llama import LlamaModel, preset
    from flextrain_b200.testing import build_llama_engine, reset_runtime
    reset_runtime()
    dev = torch.device("cuda", 0)
    cfg = preset("tiny", num_layers=4, hidden=256, num_heads=4, ffn=768, vocab=1024, seq_len=256)
    gen = torch.Generator().manual_seed(3)
    data = [torch.randint(0, cfg.vocab, (2, cfg.seq_len + 1), generator=gen) for _ in range(2)]
    dev_data = [t.to(dev) for t in data]
    it = {"i": 0}

    def batch_fn():
        t = dev_data[it["i"] % 2]
        it["i"] += 1
        return t[:, :-1], t[:, 1:]

    ft_cfg = {"batch_size": 4, "micro_batch_size": 2, "mixed_precision": {"device_dtype": "bf16"},
              "split_ratio": {"parameter": [0.5, 0.5], "optimizer": [0.5, 0.5], "checkpoint": [0.5, 0.5],
                              "gradient": [1.0, 0.0], "alpha": 0.25}}
    lr, wd, steps = 1e-3, 0.1, 5
    model, opt, eng = build_llama_engine(cfg, ft_cfg, batch_fn, lr=lr, weight_decay=wd, init_device=dev,
                                         dtype=torch.bfloat16)
    weights = eng.export_state_dict()
    got = []
    for _ in range(steps):
        r = eng.train_iteration()
        got.append(sum(float(x) for x in r) / len(r))
    eng.synchronize()
    eng.shutdown()
    reset_runtime()

    ref = LlamaModel(cfg, dtype=torch.float32)             # CPU: plain PyTorch statements, fp32
    ref.load_state_dict(weights)
    decay = [p for p in ref.parameters() if p.dim() > 1]
    no_decay = [p for p in ref.parameters() if p.dim() <= 1]
    ref_opt = torch.optim.AdamW([{"params": decay, "weight_decay": wd},
                                 {"params": no_decay, "weight_decay": 0.0}], lr=lr)
    want = []
    for _ in range(steps):
        ref_opt.zero_grad()
        total = 0.0
        for t in data:                                     # two micro-batches per step, mean gradient
            loss = ref(t[:, :-1], t[:, 1:])
            (loss / 2).backward()
            total += float(loss)
        ref_opt.step()
        want.append(total / 2)
    assert abs(got[0] - want[0]) < 5e-3, (got, want)
    assert max(abs(a - b) for a, b in zip(got, want)) < 2e-2, (got, want)
    assert want[-1] < want[0] - 0.05


def test_overflow_in_the_last_unit_to_finish_is_seen_by_the_step():
    """fp16 with dynamic loss scaling; from the second step on the gradient that enters the
    backward of unit 0 - the last unit whose reduction runs, still in flight on the optimizer
    stream when backward has been launched - is made infinite on the host side (an autograd
    function in the layer callback).  The step must be counted as skipped and the loss scale
    halved; the flags of that unit are raised on the optimizer stream after the compute
    stream has moved on, so a verdict read without waiting for that stream misses them."""
    import flextrain_b200 as ft
    from flextrain_b200.config import init_flextrain_config
    from flextrain_b200.models.llama import (LlamaBlock, LlamaModel, make_llm_funcs, make_param_groups,
                                             param_grouping, preset)
    from flextrain_b200.ops.adam import FlexTrainAdam
    from flextrain_b200.testing import reset_runtime
    reset_runtime()
    dev = torch.device("cuda", 0)
    cfg = preset("tiny", num_layers=4, hidden=256, num_heads=4, ffn=768, vocab=1024, seq_len=256)
    gen = torch.Generator().manual_seed(1)
    tok = torch.randint(0, cfg.vocab, (2, cfg.seq_len + 1), generator=gen).to(dev)
    armed = {"on": False}

    class Poison(torch.autograd.Function):
        @staticmethod
        def forward(ctx, x):
            return x.view_as(x)

        @staticmethod
        def backward(ctx, g):
            return g * float("inf") if armed["on"] else g

    ft.init_distributed(force_init=False)
    init_flextrain_config({"batch_size": 2, "micro_batch_size": 2,
                           "mixed_precision": {"device_dtype": "fp16", "dynamic_loss_scaling": True,
                                               "initial_scale_power": 10, "hysteresis": 1},
                           "split_ratio": {"parameter": [1.0, 0.0], "optimizer": [0.5, 0.5],
                                           "checkpoint": [1.0, 0.0], "gradient": [1.0, 0.0]}}, log=False)
    torch.manual_seed(0)
    with ft.Init(layer_class=LlamaBlock, num_layers=cfg.num_layers, param_grouping_func=param_grouping,
                 init_device=dev):
        model = LlamaModel(cfg, dtype=torch.float16, device=dev)
    opt = FlexTrainAdam(make_param_groups(model, 0.0), lr=1e-3)
    funcs = list(make_llm_funcs(model, lambda: (tok[:, :-1], tok[:, 1:])))
    plain_layer_forward = funcs[3]

    def layer_forward(start, end):
        run = plain_layer_forward(start, end)
        if start != 0:
            return run

        def poisoned(x, cos, sin):
            (out,) = run(x, cos, sin)
            return (Poison.apply(out),)
        return poisoned

    funcs[3] = layer_forward
    ft.set_llm_func(*funcs)
    eng = ft.initialize(model, opt, dist_init_required=False)
    eng.train_iteration()
    scale0, skipped0 = eng.loss_scale, eng.skipped_steps
    armed["on"] = True
    eng.train_iteration()
    assert eng.skipped_steps == skipped0 + 1
    assert eng.loss_scale == scale0 / 2
    armed["on"] = False
    losses = eng.train_iteration()
    assert all(float(l) == float(l) for l in losses)
    assert eng.skipped_steps == skipped0 + 1
    eng.synchronize()
    eng.shutdown()
    reset_runtime()
