"""``Init``: intercepts layer construction and hands every finished unit to the
parameter coordinator, so the full model never exists in one place.

Parity: flextrain/memory/initializer.py:1-159 (``Init`` :34-159,
``shutdown_init_context``/``restore_init_context`` :13-31).  Addition:
``init_device`` builds each layer directly on that device (``"cuda"`` makes a
70B-shape model constructible without ever holding a layer in host memory).
"""
from __future__ import annotations

import contextlib
import functools
from typing import Callable, List, Optional, Type

import torch

from ..config import get_flextrain_config
from ..utils.logging import rank0_logger

_ACTIVE: Optional["Init"] = None
_SUSPENDED = False


def shutdown_init_context():
    """Temporarily stop intercepting layer construction."""
    global _SUSPENDED
    _SUSPENDED = True


def restore_init_context():
    global _SUSPENDED
    _SUSPENDED = False


class Init:
    def __init__(self, layer_class: Type[torch.nn.Module], num_layers: int, enabled: bool = True,
                 param_grouping_func: Optional[Callable[[str, torch.nn.Parameter], int]] = None,
                 init_device=None):
        self.layer_class = layer_class
        self.num_layers = int(num_layers)
        self.enabled = enabled
        self.param_grouping_func = param_grouping_func or (lambda name, p: 0)
        self.init_device = init_device
        self._orig_init = None
        self._pending: List[torch.nn.Module] = []
        self._built = 0
        self._unit = 0
        self._interval = get_flextrain_config().checkpoint_interval

    # ---------------------------------------------------------------- enter
    def __enter__(self):
        global _ACTIVE
        if not self.enabled:
            return self
        if _ACTIVE is not None:
            raise RuntimeError("flextrain Init contexts cannot be nested or re-entered")
        _ACTIVE = self
        self._orig_init = self.layer_class.__init__
        owner = self

        @functools.wraps(self._orig_init)
        def patched(module, *args, **kwargs):
            if _SUSPENDED or _ACTIVE is not owner or getattr(module, "_ft_in_init", False):
                return owner._orig_init(module, *args, **kwargs)
            module._ft_in_init = True
            ctx = torch.device(owner.init_device) if owner.init_device is not None \
                else contextlib.nullcontext()
            with ctx:
                owner._orig_init(module, *args, **kwargs)
            del module._ft_in_init
            owner._layer_built(module)

        self.layer_class.__init__ = patched
        return self

    def _layer_built(self, module: torch.nn.Module):
        self._pending.append(module)
        self._built += 1
        if len(self._pending) == self._interval or self._built == self.num_layers:
            self._flush()

    def _flush(self):
        if not self._pending:
            return
        from .coordinator.parameter import get_para_coordinator
        params, grouping = [], []
        for layer in self._pending:
            for name, p in layer.named_parameters():
                params.append(p)
                grouping.append(int(self.param_grouping_func(name, p)))
        get_para_coordinator().init_unit_parameters(
            self.num_layers, self._unit, list(self._pending), params, grouping)
        self._unit += 1
        self._pending = []

    # ----------------------------------------------------------------- exit
    def __exit__(self, exc_type, exc, tb):
        global _ACTIVE
        if not self.enabled:
            return False
        self.layer_class.__init__ = self._orig_init
        _ACTIVE = None
        if exc_type is None:
            self._flush()
            if self._built != self.num_layers:
                rank0_logger.warning(f"Init expected {self.num_layers} layers of "
                                     f"{self.layer_class.__name__} but {self._built} were built")
            from .coordinator.parameter import get_para_coordinator
            get_para_coordinator().finish_init()
        return False
