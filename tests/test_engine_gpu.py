"""Engine on one B200: bf16 tiny Llama through the sm_100a kernels, every tier
layout must give the same training trajectory as the all-HBM layout, and the
first loss must agree with an fp32 PyTorch evaluation of the same weights."""
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
