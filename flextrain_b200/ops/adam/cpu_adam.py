"""Host Adam / AdamW over pinned fp32 state, with the device-dtype copy fused in.

Parity: flextrain/ops/adam/cpu_adam.py:1-135 (``FlexTrainCPUAdam``: defaults
lr 1e-3, betas (0.9, 0.999), eps 1e-8, weight_decay 0.01, adamw_mode True;
two fp32 states per element; ``_step`` -> ``adam_update[_copy]``).
"""
from __future__ import annotations

import itertools
from typing import Optional

import torch

from ...optimizer import FlexTrainCPUOptimizer
from ...param_group import StepContext
from ..native import dtype_code, host_lib, ptr

_ID = itertools.count()


def cpu_adam_update(step: int, lr: float, beta1: float, beta2: float, eps: float,
                    weight_decay: float, adamw_mode: bool, bias_correction: bool,
                    master: torch.Tensor, grad: torch.Tensor, exp_avg: torch.Tensor,
                    exp_avg_sq: torch.Tensor, device_copy: Optional[torch.Tensor] = None,
                    grad_scale: float = 1.0, threads: int = 0, force_scalar: bool = False) -> bool:
    """One fused Adam call on flat contiguous CPU tensors.  ``grad`` may be
    fp32, bf16 or fp16 and is multiplied by ``grad_scale`` first.  Returns True
    when a non-finite scaled gradient was met (state is then garbage: callers
    that need skip-on-overflow test the gradient before stepping)."""
    n = master.numel()
    for t in (master, grad, exp_avg, exp_avg_sq, device_copy):
        if t is None:
            continue
        if t.device.type != "cpu" or not t.is_contiguous():
            raise ValueError("cpu_adam_update needs contiguous CPU tensors")
        if t.numel() != n:
            raise ValueError("cpu_adam_update: all buffers must have the same element count")
    if master.dtype != torch.float32 or exp_avg.dtype != torch.float32 \
            or exp_avg_sq.dtype != torch.float32:
        raise TypeError("master weights and Adam moments must be fp32")
    rc = host_lib().ft_adam_update(
        int(step), float(lr), float(beta1), float(beta2), float(eps), float(weight_decay),
        int(bool(adamw_mode)), int(bool(bias_correction)), float(grad_scale),
        ptr(master), ptr(grad), dtype_code(grad.dtype), ptr(exp_avg), ptr(exp_avg_sq), n,
        ptr(device_copy), -1 if device_copy is None else dtype_code(device_copy.dtype),
        int(threads), int(force_scalar))
    if rc < 0:
        raise RuntimeError(f"ft_adam_update rejected its arguments (code {rc})")
    return rc == 1


class FlexTrainCPUAdam(FlexTrainCPUOptimizer):
    optimizer_state_per_element = 2

    def __init__(self, param_groups=None, lr: float = 1e-3, bias_correction: bool = True,
                 betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01,
                 amsgrad: bool = False, adamw_mode: bool = True, threads: int = 0):
        if amsgrad:
            raise NotImplementedError("amsgrad is not supported")
        self.defaults = dict(lr=lr, bias_correction=bias_correction, betas=tuple(betas), eps=eps,
                             weight_decay=weight_decay, amsgrad=False)
        self.adamw_mode = adamw_mode
        self.threads = threads
        self.opt_id = next(_ID)
        host_lib().ft_adam_create(self.opt_id, lr, betas[0], betas[1], eps, weight_decay,
                                  int(adamw_mode))
        super().__init__(param_groups)

    def __del__(self):
        try:
            host_lib().ft_adam_destroy(self.opt_id)
        except Exception:
            pass

    def _init_optimizer_states(self, numel: int, dtype: torch.dtype, pin: bool = False):
        make = (lambda: torch.zeros(numel, dtype=dtype).pin_memory()) if pin and \
            torch.cuda.is_available() else (lambda: torch.zeros(numel, dtype=dtype))
        return [make(), make()]

    def _step(self, ctx: StepContext, step: int, grad_scale: float = 1.0) -> bool:
        g = ctx.group
        beta1, beta2 = g.get("betas", self.defaults["betas"])
        return cpu_adam_update(
            step, g.get("lr", self.defaults["lr"]), beta1, beta2,
            g.get("eps", self.defaults["eps"]),
            g.get("weight_decay", self.defaults["weight_decay"]), self.adamw_mode,
            g.get("bias_correction", self.defaults["bias_correction"]),
            ctx.master, ctx.grad, ctx.states[0], ctx.states[1], ctx.device_copy,
            grad_scale=grad_scale, threads=self.threads)
