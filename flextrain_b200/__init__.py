"""flextrain_b200: a Blackwell-native memory-tiering LLM training engine with
the public API of FlexTrain.

Parity: flextrain/__init__.py:1-83 (``add_config_arguments`` :21-49,
``initialize`` :52-83, re-exports of ``Init``, ``set_llm_func``, ``LLMFunc``,
``init_distributed`` and the ``distributed`` module alias).

Typical use::

    import flextrain_b200 as flextrain
    from flextrain_b200.config import init_flextrain_config
    from flextrain_b200.ops.adam import FlexTrainAdam

    flextrain.init_distributed()
    init_flextrain_config(cfg_dict)
    with flextrain.Init(layer_class=Block, num_layers=L):
        model = build_model()
    opt = FlexTrainAdam(param_groups, lr=...)
    flextrain.set_llm_func(get_layer, get_batch, pre_process, layer_forward, post_process, loss)
    engine = flextrain.initialize(model, opt)
    losses = engine.train_iteration()
"""
from __future__ import annotations

import argparse
from typing import Optional

from . import defaults
from .config import get_flextrain_config, init_flextrain_config
from .llm_func import LLMFunc, set_llm_func
from .memory.initializer import Init, restore_init_context, shutdown_init_context
from .utils import distributed
from .utils.distributed import init_distributed
from .utils.logging import logger, rank0_logger

__version__ = "0.1.0"


def add_config_arguments(parser: argparse.ArgumentParser) -> argparse.ArgumentParser:
    """Add ``--flextrain`` and ``--flextrain-config <json>`` to ``parser``."""
    group = parser.add_argument_group("FlexTrain", "FlexTrain configurations")
    group.add_argument("--flextrain", default=False, action="store_true",
                       help="Enable FlexTrain (helper flag for user code, no impact on the engine)")
    group.add_argument("--flextrain-config", "--flextrain_config", default=None, type=str,
                       dest="flextrain_config", help="FlexTrain json configuration file")
    return parser


def initialize(model=None, optimizer=None, config=None, dist_init_required: Optional[bool] = None,
               dist_backend=defaults.TORCH_DISTRIBUTED_BACKEND_DEFAULT,
               timeout=defaults.PROCESS_GROUP_TIMEOUT_DEFAULT,
               init_method=defaults.TORCH_DISTRIBUTED_INIT_METHOD_DEFAULT, rank=-1, world_size=-1):
    """Wrap ``model`` and ``optimizer`` into a ``FlexTrainEngine``.

    ``config`` (dict or JSON path) initialises the config singleton when it has
    not been initialised yet - it normally has, because ``Init`` needs it."""
    from .engine import FlexTrainEngine
    if model is None or optimizer is None:
        raise ValueError("initialize() needs both a model and a FlexTrain optimizer")
    if config is not None:
        try:
            get_flextrain_config()
        except RuntimeError:
            init_flextrain_config(config)
    if dist_init_required is None or dist_init_required:
        init_distributed(dist_backend=dist_backend, timeout=timeout, init_method=init_method,
                         force_init=bool(dist_init_required), rank=rank, world_size=world_size)
    return FlexTrainEngine(model, optimizer)


_LAZY = {"FlexTrainEngine": ("engine", "FlexTrainEngine"), "FlexTrainOptimizer": ("optimizer", "FlexTrainOptimizer"),
         "op_builder": ("ops.op_builder", None), "checkpointing": ("checkpointing", None)}


def __getattr__(name):
    # names the reference package also exposes at its root (flextrain/__init__.py:5-18); resolved
    # on first use so that ``import flextrain_b200`` stays light
    if name in _LAZY:
        import importlib
        module, attr = _LAZY[name]
        mod = importlib.import_module(f"{__name__}.{module}")
        value = getattr(mod, attr) if attr else mod
        globals()[name] = value
        return value
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


__all__ = ["Init", "LLMFunc", "add_config_arguments", "distributed", "get_flextrain_config",
           "init_distributed", "init_flextrain_config", "initialize", "logger", "rank0_logger",
           "restore_init_context", "set_llm_func", "shutdown_init_context"]
