"""Step timing and throughput reporting.

The reference measures nothing per step (timers exist only inside
flextrain/auto_config.py:100-164).  ``StepTimer`` keeps wall-clock step times;
``ThroughputReporter`` turns tokens per step and a model FLOP count into
tokens/s and TFLOPS per GPU; ``cuda_timed`` brackets a callable with CUDA
events on the launching stream.
"""
from __future__ import annotations

import time
from typing import Callable, Dict, List, Optional

import torch


class StepTimer:
    def __init__(self, keep: int = 256):
        self._t0: Optional[float] = None
        self._times: List[float] = []
        self._keep = keep

    def start_step(self):
        self._t0 = time.perf_counter()

    def end_step(self):
        if self._t0 is None:
            return
        self._times.append(time.perf_counter() - self._t0)
        if len(self._times) > self._keep:
            self._times.pop(0)
        self._t0 = None

    @property
    def last(self) -> Optional[float]:
        return self._times[-1] if self._times else None

    def summary(self) -> Dict[str, Optional[float]]:
        if not self._times:
            return {"last_step_seconds": None, "mean_step_seconds": None}
        return {"last_step_seconds": self._times[-1],
                "mean_step_seconds": sum(self._times) / len(self._times)}


def llama_flops_per_token(num_layers: int, hidden: int, ffn: int, vocab: int, seq_len: int,
                          num_heads: int, num_kv_heads: Optional[int] = None,
                          recompute: bool = False) -> float:
    """Model FLOPs per token for one training step of a Llama-shape decoder:
    6 x (dense parameters touched) + causal attention score/value terms.
    ``recompute`` adds the extra forward of full activation recomputation."""
    num_kv_heads = num_kv_heads or num_heads
    head_dim = hidden // num_heads
    kv_dim = num_kv_heads * head_dim
    per_layer_params = hidden * hidden * 2 + 2 * hidden * kv_dim + 3 * hidden * ffn
    dense = num_layers * per_layer_params + hidden * vocab
    attn_fwd = num_layers * 2 * 2 * seq_len * hidden / 2     # QK^T and PV, causal half
    mult = 4.0 if recompute else 3.0
    return mult * (2.0 * dense + attn_fwd)


class ThroughputReporter:
    def __init__(self, tokens_per_step: int, flops_per_token: float, n_gpus: int):
        self.tokens_per_step = tokens_per_step
        self.flops_per_token = flops_per_token
        self.n_gpus = n_gpus

    def report(self, seconds_per_step: float) -> Dict[str, float]:
        tps = self.tokens_per_step / seconds_per_step
        return {"tokens_per_s": tps,
                "tflops_per_gpu": tps * self.flops_per_token / self.n_gpus / 1e12,
                "ms_per_step": seconds_per_step * 1e3}


def cuda_timed(fn: Callable[[], None], iters: int = 10, warmup: int = 3) -> float:
    """Mean milliseconds per call, CUDA events on the current stream, with a
    synchronise on both sides."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        fn()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / iters
