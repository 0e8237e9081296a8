"""Guard mode (FLEXTRAIN_GUARD=1): pattern bands around every runtime buffer.

The engine runs whole training steps over DRAM and NVMe tiers with the bands in place:
nothing may touch them, and the losses must equal a run without bands.  A write one
element past a buffer must be reported with the place the buffer was allocated at.
"""
import tempfile

import pytest
import torch

from flextrain_b200 import memory as M


@pytest.fixture
def guard(monkeypatch):
    monkeypatch.setenv("FLEXTRAIN_GUARD", "1")
    M.clear_guards()
    yield
    M.clear_guards()


def test_overrun_is_reported_with_its_origin(guard):
    t = M.allocate_memory(1000, torch.float32, "cpu", pinned=False, zero=True)
    assert t.numel() == 1000 and float(t.sum()) == 0.0
    assert M.check_guards() == []
    whole = M._GUARDS[-1][0]
    band = M._GUARDS[-1][1]
    # one page in front: the payload keeps whatever alignment the allocation has
    assert band == 4096 and t.data_ptr() - whole.data_ptr() == band
    # one element past the end, through a view of the whole allocation
    whole[band + 4000:band + 4004] = 0
    with pytest.raises(RuntimeError, match=r"test_guard_mode.py:\d+ .*after the buffer.*offset 4000"):
        M.check_guards()
    whole[band + 4000:band + 4004] = M._GUARD_BYTE
    whole[band - 1] = 0                                   # one byte in front
    found = M.check_guards(raise_on_damage=False)
    assert len(found) == 1 and "before the buffer" in found[0] and "offset -1" in found[0]


def test_accounting_books_the_payload_only(guard):
    before = M.allocated_bytes()["dram"]
    M.allocate_memory(10, torch.float32, "cpu", pinned=False)
    assert M.allocated_bytes()["dram"] - before == 40


def test_outside_guard_mode_nothing_is_tracked(monkeypatch):
    monkeypatch.delenv("FLEXTRAIN_GUARD", raising=False)
    M.clear_guards()
    M.allocate_memory(10, torch.float32, "cpu", pinned=False)
    assert M._GUARDS == [] and M.check_guards() == []


def _train(split, swap):
    from flextrain_b200.models.llama import preset
    from flextrain_b200.testing import build_llama_engine
    cfg = preset("tiny", num_layers=4, hidden=64, num_heads=2, ffn=136, vocab=128, seq_len=16)
    gen = torch.Generator().manual_seed(3)
    data = [torch.randint(0, 128, (2, 17), generator=gen) for _ in range(2)]
    it = {"i": 0}

    def batch_fn():
        t = data[it["i"] % 2]
        it["i"] += 1
        return t[:, :-1].contiguous(), t[:, 1:].contiguous()

    ft_cfg = {"batch_size": 4, "micro_batch_size": 2, "checkpoint_interval": 2,
              "mixed_precision": {"device_dtype": "fp32"}, "split_ratio": split,
              "nvme_swap": {"swap_dir": swap, "aio_thread_count": 2}, "engine": {"num_unit_buffers": 3}}
    model, opt, eng = build_llama_engine(cfg, ft_cfg, batch_fn, lr=1e-3, weight_decay=0.01, backend="gloo")
    losses = []
    for _ in range(3):
        out = eng.train_iteration()                        # guard mode: checks the bands itself
        losses.append(sum(float(x.detach()) for x in out) / len(out))
    eng.check_guards()
    eng.shutdown()
    return losses


SPLIT = {"parameter": [0.25, 0.5], "optimizer": [0.25, 0.5], "checkpoint": [0.25, 0.5],
         "gradient": [0.5, 0.5], "alpha": 0.25}


def test_engine_steps_leave_every_band_intact(fresh_runtime, monkeypatch):
    with tempfile.TemporaryDirectory() as swap:
        plain = _train(SPLIT, swap)
    from flextrain_b200.testing import reset_runtime
    reset_runtime()
    monkeypatch.setenv("FLEXTRAIN_GUARD", "1")
    with tempfile.TemporaryDirectory() as swap:
        guarded = _train(SPLIT, swap)
    assert len(M._GUARDS) > 10, "the runtime's buffers were expected to carry bands"
    assert max(abs(a - b) for a, b in zip(plain, guarded)) < 1e-6
