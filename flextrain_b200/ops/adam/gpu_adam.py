"""Adam on the rank's compute device.

On CUDA this is the sm_100a kernel ``ft_adam_cuda`` (fp32 master / moments,
gradient in fp32, bf16 or fp16, unscale folded in, optional device-resident
skip flag, device-dtype copy written in the same pass).  The reference has no
device-side optimizer at all (flextrain/memory/coordinator/optimizer.py:133-136
asserts the GPU share of the optimizer state to zero).  On the CPU backend the
same call runs the host kernel, so engine code is identical under gloo.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..native import cuda_lib, dtype_code, host_lib, ptr, stream_handle
from .cpu_adam import cpu_adam_update


def device_adam_update(group: Dict, step: int, defaults_owner, master: torch.Tensor,
                       grad: torch.Tensor, states: List[torch.Tensor],
                       device_copy: Optional[torch.Tensor], grad_scale: float = 1.0,
                       skip_flag: Optional[torch.Tensor] = None):
    """One fused Adam call over flat tensors that all live on one device.
    ``skip_flag`` (int32 device scalar): when non-zero the kernel leaves every
    buffer untouched (a unit whose gradients overflowed)."""
    d = defaults_owner.defaults
    beta1, beta2 = group.get("betas", d["betas"])
    lr = group.get("lr", d["lr"])
    eps = group.get("eps", d["eps"])
    wd = group.get("weight_decay", d["weight_decay"])
    bias_correction = group.get("bias_correction", d["bias_correction"])
    adamw = getattr(defaults_owner, "adamw_mode", True)
    n = master.numel()
    if n == 0:
        return
    if not master.is_cuda:
        if skip_flag is not None and int(skip_flag.item()) != 0:
            return
        cpu_adam_update(step, lr, beta1, beta2, eps, wd, adamw, bias_correction, master,
                        grad.contiguous(), states[0], states[1], device_copy, grad_scale=grad_scale)
        return
    rc = cuda_lib().ft_adam_cuda(
        ptr(master), ptr(grad), dtype_code(grad.dtype), ptr(states[0]), ptr(states[1]),
        ptr(device_copy), -1 if device_copy is None else dtype_code(device_copy.dtype), n,
        int(step), float(lr), float(beta1), float(beta2), float(eps), float(wd), int(bool(adamw)),
        int(bool(bias_correction)), float(grad_scale), ptr(skip_flag), stream_handle())
    if rc != 0:
        raise RuntimeError(f"ft_adam_cuda failed with CUDA error {rc}")


def nonfinite_flag(grad: torch.Tensor, flag: torch.Tensor, reset: bool = True):
    """Set int32 ``flag[0]`` to 1 if ``grad`` holds an inf or NaN (device side,
    no host synchronisation)."""
    if reset:
        flag.zero_()
    if grad.numel() == 0:
        return
    if grad.is_cuda:
        rc = cuda_lib().ft_check_finite(ptr(grad), dtype_code(grad.dtype), grad.numel(), ptr(flag),
                                        stream_handle())
        if rc != 0:
            raise RuntimeError(f"ft_check_finite failed with CUDA error {rc}")
    else:
        g = grad.contiguous()
        if host_lib().ft_has_nonfinite(ptr(g), dtype_code(g.dtype), g.numel(), 0):
            flag.fill_(1)


def has_nonfinite(grad: torch.Tensor) -> bool:
    flag = torch.zeros(1, dtype=torch.int32, device=grad.device)
    nonfinite_flag(grad, flag, reset=False)
    return bool(flag.item())
