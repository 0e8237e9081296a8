import torch

from flextrain_b200.config import MixedPrecisionConfig
from flextrain_b200.loss_scaler import DynamicLossScaler, LossScaler, create_loss_scaler


def test_static_scaler():
    s = LossScaler(128.0)
    s.update_scale(True)
    assert s.loss_scale == 128.0 and not s.dynamic


def test_dynamic_halves_after_hysteresis_and_doubles_after_window():
    s = DynamicLossScaler(init_scale=2 ** 16, scale_window=4, min_scale=1.0, delayed_shift=2)
    s.update_scale(True)                       # first overflow only burns hysteresis
    assert s.loss_scale == 2 ** 16 and s.cur_hysteresis == 1
    s.update_scale(True)
    assert s.loss_scale == 2 ** 15
    for _ in range(3):
        s.update_scale(False)
    assert s.loss_scale == 2 ** 15
    s.update_scale(False)                      # 4th clean step since the overflow
    assert s.loss_scale == 2 ** 16
    assert s.cur_hysteresis == 2               # refilled when the scale grows


def test_min_scale_and_consecutive_hysteresis():
    s = DynamicLossScaler(init_scale=2.0, min_scale=1.0, delayed_shift=1)
    s.update_scale(True)
    s.update_scale(True)
    assert s.loss_scale == 1.0
    c = DynamicLossScaler(init_scale=8.0, delayed_shift=2, consecutive_hysteresis=True, scale_window=100)
    c.update_scale(True)
    c.update_scale(False)                      # a clean step refills the budget
    c.update_scale(True)
    assert c.loss_scale == 8.0


def test_factory_follows_dtype_and_flags():
    assert isinstance(create_loss_scaler(MixedPrecisionConfig({"device_dtype": "fp16"})), DynamicLossScaler)
    st = create_loss_scaler(MixedPrecisionConfig({"device_dtype": "fp16", "dynamic_loss_scaling": False,
                                                  "loss_scale": 512}))
    assert isinstance(st, LossScaler) and st.loss_scale == 512
    bf = create_loss_scaler(MixedPrecisionConfig({"device_dtype": "bf16"}))
    assert isinstance(bf, LossScaler) and bf.loss_scale == 1.0
    d = create_loss_scaler(MixedPrecisionConfig({"device_dtype": "fp16", "initial_scale_power": 8}))
    assert d.loss_scale == 256.0


def test_state_dict_roundtrip_and_overflow_probe():
    s = DynamicLossScaler(init_scale=64.0)
    s.update_scale(True)
    t = DynamicLossScaler()
    t.load_state_dict(s.state_dict())
    assert t.loss_scale == s.loss_scale and t.cur_iter == s.cur_iter
    p = torch.nn.Parameter(torch.ones(3))
    p.grad = torch.tensor([1.0, float("inf"), 0.0])
    assert s.has_overflow([p])
