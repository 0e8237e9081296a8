"""Both arms of bench.py must train the same model on the same box, and the
reference arm must decline (not try) when the box cannot hold its state."""
import os
import sys
import types

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
GiB = 2 ** 30


def _fake_torch(hbm_free):
    cuda = types.SimpleNamespace(mem_get_info=lambda: (int(hbm_free), int(180 * GiB)))
    return types.SimpleNamespace(cuda=cuda)


def _fake_psutil(avail):
    return types.SimpleNamespace(virtual_memory=lambda: types.SimpleNamespace(available=avail))


def _args(**over):
    base = dict(model="auto", seq_len=0, layers=0, micro_batches_per_rank=0, unit_buffers=3, alpha=0.25)
    base.update(over)
    return types.SimpleNamespace(**base)


@pytest.mark.parametrize("world,dram_gb", [(1, 150), (1, 210), (2, 268), (4, 400), (4, 500), (4, 1006),
                                           (8, 600), (8, 1006), (8, 2000)])
def test_both_arms_choose_the_same_model(world, dram_gb):
    import bench
    from baseline import run_reference as rr
    from baseline.llama_torch import SHAPES
    dram = dram_gb * 1e9
    ours = bench.pick_model(_args(), world, int(178 * GiB), dram)[0]
    ref = rr._auto_model(world, _fake_torch(178 * GiB), _fake_psutil(dram), SHAPES, bench.MICRO_BATCH, _args())
    assert ours == ref
    # nothing of the package besides the capacity planner entered through the reference's chooser
    assert "_ft_capacity_planner" in sys.modules


def test_reference_arm_declines_what_its_host_memory_cannot_hold():
    from baseline import run_reference as rr
    from baseline.llama_torch import SHAPES
    assert rr._host_capacity_shortfall(SHAPES["llama2-13b"], _fake_psutil(210e9)) is None      # ran on such a box
    why = rr._host_capacity_shortfall(SHAPES["llama3-70b"], _fake_psutil(1006e9))
    assert why and "988 GB" in why and "1006 GB" in why
    assert rr._host_capacity_shortfall(SHAPES["llama3-70b"], _fake_psutil(1200e9)) is None


def test_debug_overrides_reach_both_choosers():
    import bench
    from baseline import run_reference as rr
    from baseline.llama_torch import SHAPES
    a = _args(layers=8)
    ours = bench.pick_model(a, 1, int(178 * GiB), 210e9)[0]
    ref = rr._auto_model(1, _fake_torch(178 * GiB), _fake_psutil(210e9), SHAPES, bench.MICRO_BATCH, a)
    assert ours == ref == "llama3-70b"          # eight 70B-shape layers fit one GPU
