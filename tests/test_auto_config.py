import pytest

from flextrain_b200.auto_config import (ConfigResult, FlexTrainConfigSolver, MachinePerfParams,
                                        format_results, trimmed_mean)
from flextrain_b200.lp import LinearProgram


def _perf(**over):
    base = dict(world_size=8, num_layers=80, opt_states=2, device_itemsize=2, gradacc_itemsize=4,
                master_itemsize=4, layer_fwd_time=0.012, layer_bwd_time=0.024, pre_post_time=0.05,
                vram_bytes=150e9, dram_bytes=180e9, nvme_bytes=50e9, unit_numel=855_654_400,
                interlayer_numel=2 * 4096 * 8192, pcie_bandwidth=50e9, nvme_read_bandwidth=2e9,
                nvme_write_bandwidth=1.8e9, cpu_adam_throughput=3e9, gpu_adam_throughput=200e9,
                nvlink_bandwidth=600e9)
    base.update(over)
    return MachinePerfParams(**base)


def test_trimmed_mean_ignores_outliers():
    assert trimmed_mean([1, 1, 1, 1, 1, 1, 1, 1, 1, 100]) == 1


@pytest.mark.parametrize("scipy_", [True, False])
def test_lp_small_problem(scipy_):
    lp = LinearProgram()
    lp.var("x", 0, 4)
    lp.var("y", 0, None)
    lp.minimise({"x": -3, "y": -5})
    lp.add_le({"y": 2}, 12)
    lp.add_le({"x": 3, "y": 2}, 18)
    sol = lp.solve(prefer_scipy=scipy_)
    assert abs(sol["x"] - 2) < 1e-6 and abs(sol["y"] - 6) < 1e-6
    bad = LinearProgram()
    bad.var("x", 0, 1)
    bad.minimise({"x": 1})
    bad.add_ge({"x": 1}, 2)
    assert bad.solve(prefer_scipy=scipy_) is None


def test_everything_fits_in_hbm_at_eight_gpus():
    """70B-shape state is 115 GiB per rank: with 150 GB usable the planner keeps
    parameters and optimizer state on the GPU (the reference cannot express this)."""
    r = FlexTrainConfigSolver(_perf(), alphas=[0.0, 0.25], max_mbpr=2)._solve_given_hypers(1, 0.25)
    assert r is not None
    assert r.split_ratio["parameter"][0] > 0.99 and r.split_ratio["optimizer"][0] > 0.99
    assert abs(r.iteration_time - (0.012 + 0.036) * 80 - 0.05) < 5e-3


def test_small_hbm_spills_to_dram_then_nvme():
    s = FlexTrainConfigSolver(_perf(world_size=1, vram_bytes=60e9, dram_bytes=150e9, nvme_bytes=2e12,
                                    num_layers=40, unit_numel=317_204_480, nvlink_bandwidth=0.0),
                              alphas=[0.0, 0.25], max_mbpr=2)
    r = s._solve_given_hypers(1, 0.25)
    assert r is not None
    g, c = r.split_ratio["optimizer"]
    assert g < 0.5 and c > 0.3
    for k in ("parameter", "optimizer", "checkpoint"):
        assert r.split_ratio[k][0] + r.split_ratio[k][1] <= 1.0 + 1e-6
    none = FlexTrainConfigSolver(_perf(world_size=1, vram_bytes=1e9, dram_bytes=1e9, nvme_bytes=0.0),
                                 max_mbpr=1)._solve_given_hypers(1, 0.0)
    assert none is None


def test_enumeration_stops_and_formats():
    results = FlexTrainConfigSolver(_perf(), alphas=[0.0, 0.25], max_mbpr=6).solve()
    assert results and all(isinstance(r, ConfigResult) for r in results)
    assert [r.micro_batches_per_rank for r in results] == list(range(1, len(results) + 1))
    text = format_results(results)
    assert "mbpr=" in text and "alpha=" in text
    cfg = results[0].to_config()
    assert set(cfg["split_ratio"]) >= {"parameter", "optimizer", "checkpoint", "gradient", "alpha"}


def test_lp_rows_in_natural_units_do_not_swallow_the_tie_break():
    """Capacity rows carry coefficients around 1e11 (bytes), the objective's tie-breaking terms are
    around 1e-4: the solver must still return the vertex with the smaller objective (it did not
    before the rows were scaled: a compute-bound step left two thirds of the optimizer state on
    the host although HBM had room)."""
    from flextrain_b200.lp import LinearProgram
    for prefer_scipy in (True, False):
        lp = LinearProgram()
        lp.var("gpu", 0.0, 1.0)
        lp.var("cpu", 0.0, 1.0)
        lp.var("T", 0.0, None)
        lp.add_eq({"gpu": 1, "cpu": 1}, 1.0)
        lp.add_le({"gpu": 1.52e11}, 1.4e11)            # HBM holds 92 % of the state
        lp.add_le({"cpu": 1.52e11}, 1.0e11)            # host memory 66 %
        lp.add_ge({"T": 1.0}, 0.065)                   # compute-bound: placement does not change T
        lp.minimise({"T": 1.0, "cpu": 3.9e-4})
        sol = lp.solve(prefer_scipy=prefer_scipy)
        assert sol is not None and abs(sol["gpu"] - 1.4e11 / 1.52e11) < 1e-6, sol
