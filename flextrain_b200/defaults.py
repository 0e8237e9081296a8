"""Config key names, their defaults and the benchmark / planner constants.

Parity: flextrain/defaults.py:1-212.  Keys and defaults are those of the
reference schema; additions for the B200 engine are grouped at the end.
"""
import os
from datetime import timedelta

import torch

# ---------------------------------------------------------------- top level
AUTO_CONFIG = "auto_config"
AUTO_CONFIG_DEFAULT = False
MAX_DRAM_USAGE = "max_dram_usage"          # GB, consumed by the planner only
BATCH_SIZE = "batch_size"                  # global
MICRO_BATCH_SIZE = "micro_batch_size"      # per GPU
CHECKPOINT_INTERVAL = "checkpoint_interval"  # layers per unit
CHECKPOINT_INTERVAL_DEFAULT = 1

# -------------------------------------------------------------- split ratios
# Every ratio is (GPU, CPU); the NVMe share is the remainder.
SPLIT_RATIO = "split_ratio"
CHECKPOINT = "checkpoint"
CHECKPOINT_DEFAULT = (0.0, 1.0)
GRADIENT = "gradient"
GRADIENT_DEFAULT = (0.0, 1.0)
PARAMETER = "parameter"
PARAMETER_DEFAULT = (0.0, 1.0)
OPTIMIZER = "optimizer"
OPTIMIZER_DEFAULT = (0.0, 1.0)
ALPHA = "alpha"
ALPHA_DEFAULT = 0.25

# ------------------------------------------------------------------ NVMe swap
NVME_SWAP = "nvme_swap"
SWAP_DIR = "swap_dir"
SWAP_DIR_DEFAULT = os.path.join(os.getcwd(), "nvme_swap")
AIO_BLOCK_SIZE = "aio_block_size"
AIO_BLOCK_SIZE_DEFAULT = 1048576
AIO_QUEUE_DEPTH = "aio_queue_depth"
AIO_QUEUE_DEPTH_DEFAULT = 8
AIO_THREAD_COUNT = "aio_thread_count"
AIO_THREAD_COUNT_DEFAULT = 4
AIO_SINGLE_SUBMIT = "aio_single_submit"
AIO_SINGLE_SUBMIT_DEFAULT = False
AIO_OVERLAP_EVENTS = "aio_overlap_events"
AIO_OVERLAP_EVENTS_DEFAULT = True
IO_ENGINE = "io_engine"                    # "io_uring" | "aio" | "psync" | "auto"
IO_ENGINE_DEFAULT = "auto"

# ------------------------------------------------------------ mixed precision
MIXED_PRECISION = "mixed_precision"
DEVICE_DTYPE = "device_dtype"
DEVICE_DTYPE_DEFAULT = torch.float16
GRADACC_DTYPE = "gradacc_dtype"
GRADACC_DTYPE_DEFAULT = torch.float32
MASTER_DTYPE = "master_dtype"
MASTER_DTYPE_DEFAULT = torch.float32
DYNAMIC_LOSS_SCALING = "dynamic_loss_scaling"
DYNAMIC_LOSS_SCALING_DEFAULT = True
INITIAL_SCALE_POWER = "initial_scale_power"
INITIAL_SCALE_POWER_DEFAULT = 16
LOSS_SCALE_WINDOW = "loss_scale_window"
LOSS_SCALE_WINDOW_DEFAULT = 1000
HYSTERESIS = "hysteresis"
HYSTERESIS_DEFAULT = 2
CONSECUTIVE_HYSTERESIS = "consecutive_hysteresis"
CONSECUTIVE_HYSTERESIS_DEFAULT = False
MIN_LOSS_SCALE = "min_loss_scale"
MIN_LOSS_SCALE_DEFAULT = 1.0
STATIC_LOSS_SCALE = "loss_scale"           # used when dynamic scaling is off
STATIC_LOSS_SCALE_DEFAULT = 1.0

# ------------------------------------------------- benchmark (auto_config)
BENCHMARK_GPU_ITERATIONS = 200
BENCHMARK_PCIE_ITERATIONS = 200
BENCHMARK_NVME_ITERATIONS = 50
BENCHMARK_CPU_ITERATIONS = 100
BENCHMARK_PCIE_BLOCK_SIZE = 2 ** 30
BENCHMARK_NVME_BLOCK_SIZE = 2 ** 32
BENCHMARK_OPTIMIZER_BLOCK_SIZE = 2 ** 28
BENCHMARK_NUM_BLOCKS = 16
ACCESSIBLE_GPU_MEMORY_RATIO = 0.99
ACCESSIBLE_CPU_MEMORY_RATIO = 0.95
POTENTIAL_ALPHA_VALUES = [0.01 * i for i in range(31)]
THROUGHPUT_STABLE_THRESHOLD = 1.01
REGULARIZATION_PENALTY = 1e-2
NUM_EXTRA_CONFIGS = 20

# ------------------------------------------------------------- distributed
PROCESS_GROUP_TIMEOUT_DEFAULT = timedelta(
    minutes=int(os.getenv("FLEXTRAIN_TIMEOUT", default=30)))
TORCH_DISTRIBUTED_BACKEND_DEFAULT = "nccl"
TORCH_DISTRIBUTED_INIT_METHOD_DEFAULT = "env://"

# ------------------------------------------------------- B200 engine additions
ENGINE = "engine"
FUSED_COLLECTIVES = "fused_collectives"    # peer-memory kernels instead of NCCL
FUSED_COLLECTIVES_DEFAULT = "auto"         # "auto" | True | False
FUSED_NONLAYER = "fused_nonlayer"          # fused all-reduce + sharded Adam for non-layerwise params
FUSED_NONLAYER_DEFAULT = "auto"            # "auto": on wherever the fused collectives are
FUSED_FIRST_GEMM = "fused_first_gemm"      # all-gather of a unit's first matrix inside the GEMM that uses it
FUSED_FIRST_GEMM_DEFAULT = "auto"          # "auto" | True | False
FUSED_BLOCKS = "fused_blocks"              # CTAs of the fused collective kernels
FUSED_BLOCKS_DEFAULT = 0                   # 0: one CTA per SM (148)
FUSED_TIMEOUT_ACTION = "fused_timeout_action"   # a cross-GPU wait of a fused kernel ran out:
FUSED_TIMEOUT_ACTION_DEFAULT = "raise"          # "raise" FusedCollectiveTimeout | "fallback" to NCCL silently
FUSED_WAIT_SECONDS = "fused_wait_seconds"  # [steady state, first step]: limit of every cross-GPU wait of
FUSED_WAIT_SECONDS_DEFAULT = (10.0, 30.0)  # the fused kernels (first-step allocations make ranks drift more)
NUM_UNIT_BUFFERS = "num_unit_buffers"      # HBM unit buffers in the gather ring
NUM_UNIT_BUFFERS_DEFAULT = 2
STRICT_OVERFLOW = "strict_overflow"        # hold every update until the step's
STRICT_OVERFLOW_DEFAULT = False            # gradients are known to be finite
CPU_ADAM_THREADS = "cpu_adam_threads"      # 0: cpu_count // world_size
CPU_ADAM_THREADS_DEFAULT = 0
NONLAYER_OPTIMIZER_DEVICE = "nonlayer_optimizer_device"  # "auto" | "gpu" | "cpu"
NONLAYER_OPTIMIZER_DEVICE_DEFAULT = "auto"
GRAD_CLIP = "gradient_clipping"            # 0 disables
GRAD_CLIP_DEFAULT = 0.0
WATCHDOG_SECONDS = "watchdog_seconds"      # 0 disables the step watchdog
NVTX = "nvtx"                              # NVTX range per (phase, unit, micro-batch)
NVTX_DEFAULT = False
PHASE_TIMING = "phase_timing"              # CUDA events at the phase boundaries of a step
PHASE_TIMING_DEFAULT = False
WATCHDOG_SECONDS_DEFAULT = 0.0

PAGE_SIZE = 4096                           # O_DIRECT alignment of every swap piece
