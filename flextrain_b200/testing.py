"""Helpers for tests and examples: reset the process-wide singletons and build
a tiny end-to-end training setup."""
from __future__ import annotations

from typing import Dict, Optional

import torch


def reset_runtime():
    """Forget config, coordinators, streams, swapper, callbacks and the process group."""
    from .config import reset_flextrain_config
    from .llm_func import reset_llm_func
    from .memory.coordinator.interlayer import reset_interlayer_coordinator
    from .memory.coordinator.optimizer import reset_opts_coordinator
    from .memory.coordinator.parameter import reset_para_coordinator
    from .memory.nvme_swapper import reset_nvme_swapper
    from .utils import distributed as dist
    from .utils.device import reset_streams
    reset_llm_func()
    reset_opts_coordinator()
    try:
        from .parallel.symm_mem import reset_flag_page
        reset_flag_page()
    except Exception:
        pass
    reset_para_coordinator()
    reset_interlayer_coordinator()
    reset_nvme_swapper()
    reset_streams()
    reset_flextrain_config()
    from .memory import clear_guards
    clear_guards()
    dist.shutdown()


def build_llama_engine(model_cfg, ft_config: Dict, batch_fn, lr=1e-3, weight_decay=0.0,
                       betas=(0.9, 0.999), eps=1e-8, adamw_mode=True, seed=0,
                       init_device=None, dtype=torch.float32, backend: Optional[str] = None):
    """Config -> Init -> model -> optimizer -> engine for a Llama-style model."""
    import flextrain_b200 as ft
    from .config import init_flextrain_config
    from .models.llama import LlamaBlock, LlamaModel, make_llm_funcs, make_param_groups, \
        param_grouping
    from .ops.adam import FlexTrainAdam
    if backend is not None:
        ft.init_distributed(dist_backend=backend, force_init=False)
    else:
        ft.init_distributed(force_init=False)
    init_flextrain_config(ft_config, log=False)
    torch.manual_seed(seed)
    with ft.Init(layer_class=LlamaBlock, num_layers=model_cfg.num_layers,
                 param_grouping_func=param_grouping, init_device=init_device):
        model = LlamaModel(model_cfg, dtype=dtype, device=init_device)
    opt = FlexTrainAdam(make_param_groups(model, weight_decay), lr=lr, betas=betas, eps=eps,
                        weight_decay=weight_decay, adamw_mode=adamw_mode)
    ft.set_llm_func(*make_llm_funcs(model, batch_fn))
    engine = ft.initialize(model, opt, dist_init_required=False)
    return model, opt, engine


def build_gpt_engine(model_cfg, ft_config: Dict, batch_fn, lr=1e-3, weight_decay=0.0,
                     betas=(0.9, 0.999), eps=1e-8, adamw_mode=True, seed=0,
                     init_device=None, dtype=torch.float32, backend: Optional[str] = None):
    """Config -> Init -> model -> optimizer -> engine for a GPT-style model."""
    import flextrain_b200 as ft
    from .config import init_flextrain_config
    from .models.gpt import GPTBlock, GPTModel, make_llm_funcs, make_param_groups, param_grouping
    from .ops.adam import FlexTrainAdam
    if backend is not None:
        ft.init_distributed(dist_backend=backend, force_init=False)
    else:
        ft.init_distributed(force_init=False)
    init_flextrain_config(ft_config, log=False)
    torch.manual_seed(seed)
    with ft.Init(layer_class=GPTBlock, num_layers=model_cfg.num_layers,
                 param_grouping_func=param_grouping, init_device=init_device):
        model = GPTModel(model_cfg, dtype=dtype, device=init_device)
    opt = FlexTrainAdam(make_param_groups(model, weight_decay), lr=lr, betas=betas, eps=eps,
                        weight_decay=weight_decay, adamw_mode=adamw_mode)
    ft.set_llm_func(*make_llm_funcs(model, batch_fn))
    engine = ft.initialize(model, opt, dist_init_required=False)
    return model, opt, engine
