"""Typed, validated view of the user's config dict, held as a process singleton.

Parity: flextrain/config.py:1-440 (SplitRatioConfig :34-98, NVMeSwapConfig
:101-174, MixedPercisionConfig :177-303, FlexTrainConfig :306-407, singleton
:410-440).  Differences, all deliberate:

* the GPU share of ``parameter`` and ``optimizer`` may be non-zero (the
  reference asserts it to 0 in parameter.py:99-102 / coordinator/optimizer.py:133-136);
* loss-scaling keys are parsed without the trailing-comma tuple slips of
  flextrain/loss_scaler.py:188-203;
* an ``engine`` section carries the knobs of the B200 runtime.
"""
from __future__ import annotations

import json
from typing import Any, Dict, Optional, Sequence, Tuple

import torch

from . import defaults as D
from .utils.logging import rank0_logger

_DTYPE_NAMES = {
    "fp16": torch.float16, "half": torch.float16, "float16": torch.float16,
    "fp32": torch.float32, "float": torch.float32, "float32": torch.float32,
    "bf16": torch.bfloat16, "bfloat16": torch.bfloat16,
}


def parse_dtype(value) -> torch.dtype:
    """Accepts a torch.dtype or one of the strings the reference accepts
    (flextrain/config.py:262-278), with an optional ``torch.`` prefix."""
    if isinstance(value, torch.dtype):
        return value
    if isinstance(value, str):
        key = value.strip().lower()
        if key.startswith("torch."):
            key = key[len("torch."):]
        if key in _DTYPE_NAMES:
            return _DTYPE_NAMES[key]
    raise ValueError(f"unrecognised dtype specification: {value!r}")


def _ratio_pair(value, name: str, default: Tuple[float, float]) -> Tuple[float, float]:
    if value is None:
        value = default
    if isinstance(value, (int, float)):
        value = (float(value), 1.0 - float(value))
    if not isinstance(value, Sequence) or len(value) not in (2, 3):
        raise ValueError(f"split_ratio.{name} must be (GPU, CPU[, NVMe]), got {value!r}")
    gpu, cpu = float(value[0]), float(value[1])
    if gpu < 0 or cpu < 0 or gpu + cpu > 1.0 + 1e-9:
        raise ValueError(f"split_ratio.{name}: shares must be >= 0 and sum to <= 1, got {value!r}")
    if len(value) == 3 and abs(gpu + cpu + float(value[2]) - 1.0) > 1e-6:
        raise ValueError(f"split_ratio.{name}: three shares must sum to 1, got {value!r}")
    return (gpu, cpu)


class _Section:
    """``to_log(indent)``: the section as the reference prints it inside its configuration
    dump (flextrain/config.py:88-98,161-174,285-303): ``"name": {...}`` with tab indentation."""
    _SECTION_NAME = ""

    def to_log(self, indent: int = 0) -> str:
        tabs = "\t" * indent
        body = json.dumps(self.to_dict(), indent="\t", default=str).replace("\n", "\n" + tabs)
        return f'{tabs}"{self._SECTION_NAME}": {body}'


class SplitRatioConfig(_Section):
    """Where each kind of state lives.  Every entry is ``(GPU, CPU)``; NVMe
    gets ``1 - GPU - CPU``.  ``alpha`` is the fraction of every unit's
    host-side optimizer work that may be finished lazily during the next
    iteration's forward pass."""

    def __init__(self, section: Optional[Dict[str, Any]] = None):
        section = dict(section or {})
        self.checkpoint = _ratio_pair(section.get(D.CHECKPOINT), D.CHECKPOINT, D.CHECKPOINT_DEFAULT)
        self.gradient = _ratio_pair(section.get(D.GRADIENT), D.GRADIENT, D.GRADIENT_DEFAULT)
        self.parameter = _ratio_pair(section.get(D.PARAMETER), D.PARAMETER, D.PARAMETER_DEFAULT)
        self.optimizer = _ratio_pair(section.get(D.OPTIMIZER), D.OPTIMIZER, D.OPTIMIZER_DEFAULT)
        if abs(sum(self.gradient) - 1.0) > 1e-6:
            raise ValueError("split_ratio.gradient has no NVMe tier: GPU + CPU must be 1")
        alpha = section.get(D.ALPHA, D.ALPHA_DEFAULT)
        if isinstance(alpha, Sequence):      # the reference stores alpha as a 1-list
            alpha = alpha[0]
        self.alpha = float(alpha)
        if not 0.0 <= self.alpha <= 0.5:
            raise ValueError(f"split_ratio.alpha must lie in [0, 0.5], got {self.alpha}")

    @staticmethod
    def nvme_share(pair: Tuple[float, float]) -> float:
        return max(0.0, 1.0 - pair[0] - pair[1])

    def uses_nvme(self) -> bool:
        return any(self.nvme_share(p) > 1e-9
                   for p in (self.checkpoint, self.parameter, self.optimizer))

    def to_dict(self):
        return {D.CHECKPOINT: list(self.checkpoint), D.GRADIENT: list(self.gradient),
                D.PARAMETER: list(self.parameter), D.OPTIMIZER: list(self.optimizer),
                D.ALPHA: self.alpha}

    def __repr__(self):
        return f"SplitRatioConfig({self.to_dict()})"


class NVMeSwapConfig(_Section):
    def __init__(self, section: Optional[Dict[str, Any]] = None):
        section = dict(section or {})
        self.swap_dir = section.get(D.SWAP_DIR, D.SWAP_DIR_DEFAULT)
        self.aio_block_size = int(section.get(D.AIO_BLOCK_SIZE, D.AIO_BLOCK_SIZE_DEFAULT))
        self.aio_queue_depth = int(section.get(D.AIO_QUEUE_DEPTH, D.AIO_QUEUE_DEPTH_DEFAULT))
        self.aio_thread_count = int(section.get(D.AIO_THREAD_COUNT, D.AIO_THREAD_COUNT_DEFAULT))
        self.aio_single_submit = bool(section.get(D.AIO_SINGLE_SUBMIT, D.AIO_SINGLE_SUBMIT_DEFAULT))
        self.aio_overlap_events = bool(section.get(D.AIO_OVERLAP_EVENTS, D.AIO_OVERLAP_EVENTS_DEFAULT))
        self.io_engine = str(section.get(D.IO_ENGINE, D.IO_ENGINE_DEFAULT))
        if self.aio_block_size % D.PAGE_SIZE:
            raise ValueError("nvme_swap.aio_block_size must be a multiple of 4096")
        if self.aio_queue_depth < 1 or self.aio_thread_count < 1:
            raise ValueError("nvme_swap queue depth and thread count must be >= 1")
        if self.io_engine not in ("auto", "io_uring", "aio", "psync"):
            raise ValueError(f"nvme_swap.io_engine: unknown engine {self.io_engine!r}")

    def to_dict(self):
        return dict(vars(self))

    def __repr__(self):
        return f"NVMeSwapConfig({self.to_dict()})"


class MixedPrecisionConfig(_Section):
    def __init__(self, section: Optional[Dict[str, Any]] = None):
        section = dict(section or {})
        self.device_dtype = parse_dtype(section.get(D.DEVICE_DTYPE, D.DEVICE_DTYPE_DEFAULT))
        self.gradacc_dtype = parse_dtype(section.get(D.GRADACC_DTYPE, D.GRADACC_DTYPE_DEFAULT))
        self.master_dtype = parse_dtype(section.get(D.MASTER_DTYPE, D.MASTER_DTYPE_DEFAULT))
        if self.master_dtype != torch.float32:
            raise ValueError("master_dtype must be fp32: the Adam kernels keep fp32 state")
        self.dynamic_loss_scaling = bool(section.get(D.DYNAMIC_LOSS_SCALING, D.DYNAMIC_LOSS_SCALING_DEFAULT))
        self.initial_scale_power = int(section.get(D.INITIAL_SCALE_POWER, D.INITIAL_SCALE_POWER_DEFAULT))
        self.loss_scale_window = int(section.get(D.LOSS_SCALE_WINDOW, D.LOSS_SCALE_WINDOW_DEFAULT))
        self.hysteresis = int(section.get(D.HYSTERESIS, D.HYSTERESIS_DEFAULT))
        self.consecutive_hysteresis = bool(section.get(D.CONSECUTIVE_HYSTERESIS, D.CONSECUTIVE_HYSTERESIS_DEFAULT))
        self.min_loss_scale = float(section.get(D.MIN_LOSS_SCALE, D.MIN_LOSS_SCALE_DEFAULT))
        self.loss_scale = float(section.get(D.STATIC_LOSS_SCALE, D.STATIC_LOSS_SCALE_DEFAULT))

    @property
    def initial_dynamic_scale(self) -> float:
        return 2.0 ** self.initial_scale_power

    def to_dict(self):
        out = dict(vars(self))
        for k in (D.DEVICE_DTYPE, D.GRADACC_DTYPE, D.MASTER_DTYPE):
            out[k] = str(out[k])
        return out

    def __repr__(self):
        return f"MixedPrecisionConfig({self.to_dict()})"


# The reference spells the class "MixedPercisionConfig" (flextrain/config.py:177).
MixedPercisionConfig = MixedPrecisionConfig


class EngineConfig(_Section):
    """Knobs of the B200 runtime that have no counterpart in the reference."""

    def __init__(self, section: Optional[Dict[str, Any]] = None):
        section = dict(section or {})
        self.fused_collectives = section.get(D.FUSED_COLLECTIVES, D.FUSED_COLLECTIVES_DEFAULT)
        if self.fused_collectives not in ("auto", True, False):
            raise ValueError("engine.fused_collectives must be 'auto', true or false")
        self.num_unit_buffers = int(section.get(D.NUM_UNIT_BUFFERS, D.NUM_UNIT_BUFFERS_DEFAULT))
        if self.num_unit_buffers < 2:
            raise ValueError("engine.num_unit_buffers must be >= 2 (one computing, one in flight)")
        self.strict_overflow = bool(section.get(D.STRICT_OVERFLOW, D.STRICT_OVERFLOW_DEFAULT))
        self.cpu_adam_threads = int(section.get(D.CPU_ADAM_THREADS, D.CPU_ADAM_THREADS_DEFAULT))
        self.nonlayer_optimizer_device = str(section.get(
            D.NONLAYER_OPTIMIZER_DEVICE, D.NONLAYER_OPTIMIZER_DEVICE_DEFAULT))
        if self.nonlayer_optimizer_device not in ("auto", "gpu", "cpu"):
            raise ValueError("engine.nonlayer_optimizer_device must be auto|gpu|cpu")
        self.gradient_clipping = float(section.get(D.GRAD_CLIP, D.GRAD_CLIP_DEFAULT))
        self.watchdog_seconds = float(section.get(D.WATCHDOG_SECONDS, D.WATCHDOG_SECONDS_DEFAULT))
        self.nvtx = bool(section.get(D.NVTX, D.NVTX_DEFAULT))
        self.phase_timing = bool(section.get(D.PHASE_TIMING, D.PHASE_TIMING_DEFAULT))
        self.fused_blocks_setting = int(section.get(D.FUSED_BLOCKS, D.FUSED_BLOCKS_DEFAULT))
        waits = section.get(D.FUSED_WAIT_SECONDS, D.FUSED_WAIT_SECONDS_DEFAULT)
        if isinstance(waits, (int, float)):
            waits = (waits, waits)
        if len(waits) != 2 or min(waits) <= 0:
            raise ValueError("engine.fused_wait_seconds must be a positive number or [steady, first step]")
        self.fused_wait_seconds = (float(waits[0]), float(waits[1]))
        self.fused_nonlayer = section.get(D.FUSED_NONLAYER, D.FUSED_NONLAYER_DEFAULT)
        self.fused_timeout_action = str(section.get(D.FUSED_TIMEOUT_ACTION, D.FUSED_TIMEOUT_ACTION_DEFAULT))
        if self.fused_timeout_action not in ("raise", "fallback"):
            raise ValueError("engine.fused_timeout_action must be 'raise' or 'fallback'")
        self.fused_first_gemm = section.get(D.FUSED_FIRST_GEMM, D.FUSED_FIRST_GEMM_DEFAULT)
        if self.fused_first_gemm not in ("auto", True, False):
            raise ValueError("engine.fused_first_gemm must be 'auto', true or false")
        if self.fused_nonlayer not in ("auto", True, False):
            raise ValueError("engine.fused_nonlayer must be 'auto', true or false")

    @property
    def fused_blocks(self) -> int:
        """CTAs of the fused collective kernels.  Unset (0): one per SM (148), which fits
        beside a resident GEMM CTA and keeps enough peer requests in flight to fill the link."""
        return self.fused_blocks_setting if self.fused_blocks_setting > 0 else 148

    def to_dict(self):
        return dict(vars(self), fused_blocks=self.fused_blocks)

    def __repr__(self):
        return f"EngineConfig({self.to_dict()})"


SplitRatioConfig._SECTION_NAME = D.SPLIT_RATIO
NVMeSwapConfig._SECTION_NAME = D.NVME_SWAP
MixedPrecisionConfig._SECTION_NAME = D.MIXED_PRECISION
EngineConfig._SECTION_NAME = D.ENGINE


class FlexTrainConfig:
    """Whole configuration.  ``batch_size`` and ``micro_batch_size`` are required;
    ``max_dram_usage`` (GB) is required only when ``auto_config`` is on, since
    the planner is its only consumer (flextrain/config.py:358-371)."""

    def __init__(self, cfg: Dict[str, Any]):
        if isinstance(cfg, str):
            with open(cfg) as f:
                cfg = json.load(f)
        if not isinstance(cfg, dict):
            raise TypeError("config must be a dict or a path to a JSON file")
        for key in (D.BATCH_SIZE, D.MICRO_BATCH_SIZE):
            if key not in cfg:
                raise KeyError(f"config key {key!r} is required")
        self.auto_config = bool(cfg.get(D.AUTO_CONFIG, D.AUTO_CONFIG_DEFAULT))
        self.max_dram_usage = float(cfg.get(D.MAX_DRAM_USAGE, 0.0))
        if self.auto_config and self.max_dram_usage <= 0:
            raise KeyError("config key 'max_dram_usage' (GB) is required with auto_config")
        self.batch_size = int(cfg[D.BATCH_SIZE])
        self.micro_batch_size = int(cfg[D.MICRO_BATCH_SIZE])
        if self.batch_size <= 0 or self.micro_batch_size <= 0:
            raise ValueError("batch_size and micro_batch_size must be positive")
        if self.batch_size % self.micro_batch_size:
            raise ValueError("batch_size must be a multiple of micro_batch_size")
        self.checkpoint_interval = int(cfg.get(D.CHECKPOINT_INTERVAL, D.CHECKPOINT_INTERVAL_DEFAULT))
        if self.checkpoint_interval < 1:
            raise ValueError("checkpoint_interval must be >= 1")
        self.split_ratio = SplitRatioConfig(cfg.get(D.SPLIT_RATIO))
        self.nvme_swap = NVMeSwapConfig(cfg.get(D.NVME_SWAP))
        self.mixed_precision = MixedPrecisionConfig(cfg.get(D.MIXED_PRECISION))
        self.engine = EngineConfig(cfg.get(D.ENGINE))

    def micro_batches_per_rank(self, world_size: int) -> int:
        per_step = self.batch_size // self.micro_batch_size
        if per_step % world_size:
            raise ValueError(
                f"batch_size/micro_batch_size = {per_step} micro-batches cannot be "
                f"shared evenly by {world_size} ranks")
        return per_step // world_size

    def to_dict(self):
        return {
            D.AUTO_CONFIG: self.auto_config, D.MAX_DRAM_USAGE: self.max_dram_usage,
            D.BATCH_SIZE: self.batch_size, D.MICRO_BATCH_SIZE: self.micro_batch_size,
            D.CHECKPOINT_INTERVAL: self.checkpoint_interval,
            D.SPLIT_RATIO: self.split_ratio.to_dict(), D.NVME_SWAP: self.nvme_swap.to_dict(),
            D.MIXED_PRECISION: self.mixed_precision.to_dict(), D.ENGINE: self.engine.to_dict(),
        }

    def log(self):
        rank0_logger.info("FlexTrain-B200 configuration:\n" +
                          json.dumps(self.to_dict(), indent=2, default=str))


_CONFIG: Optional[FlexTrainConfig] = None


def init_flextrain_config(cfg: Dict[str, Any], log: bool = True) -> FlexTrainConfig:
    """Build the singleton.  Must run before ``Init`` is entered."""
    global _CONFIG
    _CONFIG = FlexTrainConfig(cfg)
    if log:
        _CONFIG.log()
    return _CONFIG


def get_flextrain_config() -> FlexTrainConfig:
    if _CONFIG is None:
        raise RuntimeError("FlexTrain config is not initialised: call init_flextrain_config(dict) first")
    return _CONFIG


def reset_flextrain_config():
    """Drop the singleton (tests and re-initialisation in one process)."""
    global _CONFIG
    _CONFIG = None
