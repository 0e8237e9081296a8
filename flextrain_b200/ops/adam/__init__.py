"""``FlexTrainAdam``: the optimizer object a user constructs.

Parity: flextrain/ops/adam/__init__.py:8-34 (glue of ``FlexTrainCPUAdam`` and
``FlexTrainOptimizer``).
"""
from ...optimizer import FlexTrainOptimizer
from .cpu_adam import FlexTrainCPUAdam, cpu_adam_update


class FlexTrainAdam(FlexTrainOptimizer):
    def __init__(self, param_groups, lr=1e-3, bias_correction=True, betas=(0.9, 0.999), eps=1e-8,
                 weight_decay=0.01, amsgrad=False, adamw_mode=True):
        cpu_opt = FlexTrainCPUAdam(lr=lr, bias_correction=bias_correction, betas=betas, eps=eps,
                                   weight_decay=weight_decay, amsgrad=amsgrad,
                                   adamw_mode=adamw_mode)
        super().__init__(param_groups, cpu_opt)


__all__ = ["FlexTrainAdam", "FlexTrainCPUAdam", "cpu_adam_update"]
