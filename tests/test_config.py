import json

import pytest
import torch

from flextrain_b200.config import (FlexTrainConfig, MixedPercisionConfig, MixedPrecisionConfig,
                                   get_flextrain_config, init_flextrain_config, parse_dtype,
                                   reset_flextrain_config)


def test_defaults_match_the_reference_schema():
    c = FlexTrainConfig({"batch_size": 8, "micro_batch_size": 2})
    assert c.checkpoint_interval == 1 and not c.auto_config
    assert c.split_ratio.checkpoint == (0.0, 1.0) and c.split_ratio.alpha == 0.25
    assert c.nvme_swap.aio_block_size == 1048576 and c.nvme_swap.aio_queue_depth == 8
    assert c.nvme_swap.aio_thread_count == 4 and c.nvme_swap.aio_overlap_events
    mp = c.mixed_precision
    assert mp.device_dtype == torch.float16 and mp.gradacc_dtype == torch.float32
    assert mp.initial_scale_power == 16 and mp.loss_scale_window == 1000 and mp.hysteresis == 2
    assert c.micro_batches_per_rank(2) == 2
    assert MixedPercisionConfig is MixedPrecisionConfig


@pytest.mark.parametrize("s,dt", [("fp16", torch.float16), ("half", torch.float16),
                                  ("torch.float16", torch.float16), ("fp32", torch.float32),
                                  ("float", torch.float32), ("bf16", torch.bfloat16),
                                  ("torch.bfloat16", torch.bfloat16), (torch.float32, torch.float32)])
def test_dtype_strings(s, dt):
    assert parse_dtype(s) == dt


def test_validation():
    with pytest.raises(KeyError):
        FlexTrainConfig({"batch_size": 8})
    with pytest.raises(ValueError):
        FlexTrainConfig({"batch_size": 7, "micro_batch_size": 2})
    with pytest.raises(ValueError):
        FlexTrainConfig({"batch_size": 8, "micro_batch_size": 2, "split_ratio": {"alpha": 0.75}})
    with pytest.raises(ValueError):
        FlexTrainConfig({"batch_size": 8, "micro_batch_size": 2, "split_ratio": {"parameter": [0.7, 0.7]}})
    with pytest.raises(ValueError):
        FlexTrainConfig({"batch_size": 8, "micro_batch_size": 2, "split_ratio": {"gradient": [0.3, 0.3]}})
    with pytest.raises(KeyError):
        FlexTrainConfig({"batch_size": 8, "micro_batch_size": 2, "auto_config": True})
    with pytest.raises(ValueError):
        FlexTrainConfig({"batch_size": 6, "micro_batch_size": 2}).micro_batches_per_rank(2)
    with pytest.raises(ValueError):
        parse_dtype("int8")


def test_gpu_shares_are_allowed_and_alpha_list_form():
    c = FlexTrainConfig({"batch_size": 4, "micro_batch_size": 1,
                         "split_ratio": {"parameter": [0.5, 0.25], "optimizer": [1.0, 0.0], "alpha": [0.1]}})
    assert c.split_ratio.parameter == (0.5, 0.25)
    assert abs(c.split_ratio.nvme_share(c.split_ratio.parameter) - 0.25) < 1e-9
    assert c.split_ratio.uses_nvme() and c.split_ratio.alpha == 0.1


def test_singleton_and_json_path(tmp_path):
    reset_flextrain_config()
    with pytest.raises(RuntimeError):
        get_flextrain_config()
    path = tmp_path / "c.json"
    path.write_text(json.dumps({"batch_size": 2, "micro_batch_size": 1}))
    c = init_flextrain_config(str(path), log=False)
    assert get_flextrain_config() is c
    assert json.loads(json.dumps(c.to_dict(), default=str))["batch_size"] == 2
    reset_flextrain_config()


def test_fused_wait_limits():
    base = {"batch_size": 4, "micro_batch_size": 1}
    assert FlexTrainConfig(base).engine.fused_wait_seconds == (10.0, 30.0)
    assert FlexTrainConfig({**base, "engine": {"fused_wait_seconds": 5}}).engine.fused_wait_seconds == (5.0, 5.0)
    assert FlexTrainConfig({**base, "engine": {"fused_wait_seconds": [8, 20]}}).engine.fused_wait_seconds == (8.0, 20.0)
    with pytest.raises(ValueError):
        FlexTrainConfig({**base, "engine": {"fused_wait_seconds": [1, 0]}})


def test_wait_limit_reaches_the_native_library():
    """The setter converts seconds to clock cycles and hands them to both kernel families
    (no GPU needed: the library only stores the number)."""
    import ctypes
    from flextrain_b200.ops.native import cuda_lib
    from flextrain_b200.parallel import fused
    lib = cuda_lib()
    lib.ft_comm_spin_budget.restype = ctypes.c_longlong
    try:
        cycles = fused.set_wait_seconds(30.0)
        assert 30 * 1.0e9 < cycles < 30 * 3.0e9 and lib.ft_comm_spin_budget() == cycles
        assert fused.set_wait_seconds(10.0) * 3 == cycles
    finally:
        lib.ft_comm_set_spin_budget(0)
        lib.ft_ag_set_spin_budget(0)


def test_sections_print_like_the_reference_dump():
    from flextrain_b200.config import FlexTrainConfig
    cfg = FlexTrainConfig({"batch_size": 4, "micro_batch_size": 2})
    text = cfg.split_ratio.to_log(indent=1)
    assert text.startswith('\t"split_ratio": {') and '\n\t\t"alpha": 0.25' in text and text.endswith("\n\t}")
    assert cfg.mixed_precision.to_log().startswith('"mixed_precision": {')
    assert '"aio_queue_depth": 8' in cfg.nvme_swap.to_log()
