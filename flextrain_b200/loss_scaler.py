"""Static and dynamic loss scaling.

Parity: flextrain/loss_scaler.py:1-204 (LossScalerBase/LossScaler/
DynamicLossScaler :30-179, create_loss_scaler :184-204).  Unlike the reference,
the engine really consumes this state machine: gradients are unscaled inside
the reduce-scatter/Adam kernels, their finite flag is OR-ed over units and
ranks, and ``update_scale(overflow)`` runs once per step.

State machine of the dynamic scaler
  * overflow: ``hysteresis`` counts down; once it is exhausted every further
    overflow halves the scale (never below ``min_scale``); the clean-step
    counter restarts.
  * ``scale_window`` clean steps in a row double the scale and, unless
    ``consecutive_hysteresis`` is set, refill the hysteresis budget.  With
    ``consecutive_hysteresis`` the budget refills on every clean step instead.
"""
from __future__ import annotations

import torch

from .utils.logging import rank0_logger


# keyword names of the dynamic scaler's arguments (flextrain/loss_scaler.py:15-19)
INITIAL_LOSS_SCALE = "init_scale"
SCALE_WINDOW = "scale_window"
DELAYED_SHIFT = "delayed_shift"
CONSECUTIVE_HYSTERESIS = "consecutive_hysteresis"
MIN_LOSS_SCALE = "min_scale"


def to_python_float(value) -> float:
    """One-element tensor (or number) -> Python float (flextrain/loss_scaler.py:23-27)."""
    if hasattr(value, "item"):
        return float(value.item())
    return float(value)


class LossScalerBase:
    def __init__(self, cur_scale: float):
        self.cur_scale = float(cur_scale)
        self.dynamic = False

    @property
    def loss_scale(self) -> float:
        return self.cur_scale

    def scale_gradient(self, module, grad_in, grad_out):
        return tuple(self.loss_scale * g for g in grad_in)

    def update_scale(self, overflow: bool):
        pass

    def backward(self, loss: torch.Tensor, retain_graph: bool = False):
        (loss * self.loss_scale).backward(retain_graph=retain_graph)

    def state_dict(self):
        return {"cur_scale": self.cur_scale}

    def load_state_dict(self, state):
        self.cur_scale = float(state["cur_scale"])


class LossScaler(LossScalerBase):
    """A fixed scale.  Overflowing steps are still skipped by the engine."""

    def __init__(self, scale: float = 1.0):
        super().__init__(scale)

    def has_overflow(self, params) -> bool:
        return False


class DynamicLossScaler(LossScalerBase):
    def __init__(self, init_scale: float = 2.0 ** 16, scale_factor: float = 2.0,
                 scale_window: int = 1000, min_scale: float = 1.0,
                 delayed_shift: int = 1, consecutive_hysteresis: bool = False,
                 raise_error_at_min_scale: bool = False, dtype=None):
        # ``dtype`` is accepted for call compatibility (flextrain/loss_scaler.py:104-113 stores it
        # and never reads it); the scale itself is a Python float here
        super().__init__(init_scale)
        self.dynamic = True
        self.cur_iter = 0
        self.last_overflow_iter = -1
        self.scale_factor = float(scale_factor)
        self.scale_window = int(scale_window)
        self.min_scale = float(min_scale)
        self.delayed_shift = int(delayed_shift)
        self.cur_hysteresis = int(delayed_shift)
        self.consecutive_hysteresis = bool(consecutive_hysteresis)
        self.raise_error_at_min_scale = bool(raise_error_at_min_scale)

    @staticmethod
    def _has_inf_or_nan(x: torch.Tensor) -> bool:
        return not bool(torch.isfinite(x.float().sum()))

    def has_overflow(self, params) -> bool:
        return any(p.grad is not None and self._has_inf_or_nan(p.grad) for p in params)

    def update_scale(self, overflow: bool):
        if overflow:
            if self.delayed_shift == 1 or self.cur_hysteresis == 1:
                if self.cur_scale == self.min_scale and self.raise_error_at_min_scale:
                    raise FloatingPointError("loss scale is at its minimum and gradients still overflow")
                new_scale = max(self.cur_scale / self.scale_factor, self.min_scale)
                rank0_logger.info(f"gradient overflow: loss scale {self.cur_scale:g} -> {new_scale:g}")
                self.cur_scale = new_scale
            else:
                rank0_logger.info(f"gradient overflow: hysteresis {self.cur_hysteresis} -> "
                                  f"{self.cur_hysteresis - 1}, scale stays {self.cur_scale:g}")
                self.cur_hysteresis -= 1
            self.last_overflow_iter = self.cur_iter
        else:
            if self.consecutive_hysteresis:
                self.cur_hysteresis = self.delayed_shift
            if (self.cur_iter - self.last_overflow_iter) % self.scale_window == 0:
                if not self.consecutive_hysteresis:
                    self.cur_hysteresis = self.delayed_shift
                self.cur_scale *= self.scale_factor
        self.cur_iter += 1

    def state_dict(self):
        return {k: getattr(self, k) for k in
                ("cur_scale", "cur_iter", "last_overflow_iter", "cur_hysteresis")}

    def load_state_dict(self, state):
        for k, v in state.items():
            setattr(self, k, v)


def create_loss_scaler(mixed_precision=None) -> LossScalerBase:
    """fp16 + ``dynamic_loss_scaling`` -> DynamicLossScaler; fp16 without it ->
    the configured static scale; bf16/fp32 -> static scale (1.0 by default)."""
    if mixed_precision is None:
        from .config import get_flextrain_config
        mixed_precision = get_flextrain_config().mixed_precision
    mp = mixed_precision
    if mp.device_dtype == torch.float16 and mp.dynamic_loss_scaling:
        return DynamicLossScaler(init_scale=mp.initial_dynamic_scale,
                                 scale_window=mp.loss_scale_window,
                                 min_scale=mp.min_loss_scale,
                                 delayed_shift=mp.hysteresis,
                                 consecutive_hysteresis=mp.consecutive_hysteresis)
    return LossScaler(mp.loss_scale)
