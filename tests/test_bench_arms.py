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
    base = dict(model="auto", seq_len=0, layers=0, micro_batches_per_rank=0, unit_buffers=3, alpha=0.25,
                nvme_gib_per_rank=0.0)
    base.update(over)
    return types.SimpleNamespace(**base)


@pytest.mark.parametrize("node_gpus,dram_gb", [(1, 150), (1, 196), (1, 400), (8, 600), (8, 1006), (8, 2000),
                                               (4, 500), (2, 268)])
def test_both_arms_choose_the_same_model_for_the_node(node_gpus, dram_gb):
    import bench
    from baseline import run_reference as rr
    from baseline.llama_torch import SHAPES
    dram = dram_gb * 1e9
    ours = bench.pick_model(_args(), int(178 * GiB), dram, node_gpus)[0]
    policy = {"dram_share_use": bench.DRAM_SHARE_USE, "dram_per_rank_cap": bench.DRAM_PER_RANK_CAP}
    ref = rr._auto_model(node_gpus, _fake_torch(178 * GiB), _fake_psutil(dram), SHAPES, bench.MICRO_BATCH,
                         _args(), policy)
    assert ours == ref
    # nothing of the package besides the capacity planner entered through the reference's chooser
    assert "_ft_capacity_planner" in sys.modules


def test_one_model_per_node_whatever_the_number_of_ranks():
    """A one-GPU box (196 GB of host memory) and one GPU of an eight-GPU box (1006 GB shared by
    eight) must train the same model with the same host-memory budget, or the scaling curve and
    the single-GPU record describe different benchmarks."""
    import bench
    small = bench.pick_model(_args(), int(178 * GiB), 196e9, 1)[0]
    big = bench.pick_model(_args(), int(178 * GiB), 1006e9, 8)[0]
    assert small == big == "llama2-13b"
    assert bench.dram_per_rank(196e9, 1) == bench.dram_per_rank(1006e9, 8) == bench.DRAM_PER_RANK_CAP
    # and the split of that model exists at every N
    for n in (1, 2, 4, 8):
        assert bench.plan_split(_args(nvme_gib_per_rank=0.0), "llama2-13b", n, int(178 * GiB), 1006e9, 8)
    # the 70B shape needs the eight GPUs together
    assert bench.plan_split(_args(nvme_gib_per_rank=0.0), "llama3-70b", 8, int(178 * GiB), 1006e9, 8)
    assert bench.plan_split(_args(nvme_gib_per_rank=0.0), "llama3-70b", 1, int(178 * GiB), 1006e9, 8) is None


def test_reference_arm_declines_what_its_host_memory_cannot_hold():
    from baseline import run_reference as rr
    from baseline.llama_torch import SHAPES
    assert rr._host_capacity_shortfall(SHAPES["llama2-13b"], _fake_psutil(210e9)) is None      # ran on such a box
    why = rr._host_capacity_shortfall(SHAPES["llama3-70b"], _fake_psutil(1006e9))
    assert why and "988 GB" in why and "1006 GB" in why
    assert rr._host_capacity_shortfall(SHAPES["llama3-70b"], _fake_psutil(1200e9)) is None
    # on a box shared with other GPUs' users the arm declines much earlier
    assert rr._host_capacity_shortfall(SHAPES["llama2-13b"], _fake_psutil(1006e9), whole_box=False) is None
    assert rr._host_capacity_shortfall(SHAPES["llama3-70b"], _fake_psutil(1500e9), whole_box=False)


def test_reference_alpha_is_one_the_reference_accepts():
    """13B keeps the 0.25 both arms were measured with; the 70B shape at one rank needs less."""
    from baseline import run_reference as rr
    from baseline.llama_torch import SHAPES
    for world in (1, 2, 4, 8):
        assert rr._feasible_alpha(SHAPES["llama2-13b"], world, 8, 1, 0.25) == 0.25
    a = rr._feasible_alpha(SHAPES["llama3-70b"], 1, 2, 1, 0.25)
    assert 0 < a < 0.07843
    assert rr._feasible_alpha(SHAPES["llama3-70b"], 8, 2, 1, 0.25) == 0.25


def test_debug_overrides_reach_both_choosers():
    import bench
    from baseline import run_reference as rr
    from baseline.llama_torch import SHAPES
    a = _args(layers=8)
    ours = bench.pick_model(a, int(178 * GiB), 210e9, 1)[0]
    ref = rr._auto_model(1, _fake_torch(178 * GiB), _fake_psutil(210e9), SHAPES, bench.MICRO_BATCH, a)
    assert ours == ref == "llama3-70b"          # eight 70B-shape layers fit one GPU


def test_extra_model_only_where_it_is_wanted():
    import bench
    a = bench.parse_args([])
    assert not bench._wants_extra(a, 1) and not bench._wants_extra(a, 4) and bench._wants_extra(a, 8)
    assert not bench._wants_extra(bench.parse_args(["--extra", "off"]), 8)
    assert not bench._wants_extra(bench.parse_args(["--model", "llama2-7b"]), 8)
    assert bench._wants_extra(bench.parse_args(["--model", "llama2-7b", "--extra", "on"]), 2)
    assert not bench._wants_extra(bench.parse_args(["--as-extra", "--model", "llama3-70b"]), 8)
