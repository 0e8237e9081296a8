"""Activation checkpointing with exact RNG replay, plus a Megatron-style CUDA
RNG tracker.

Parity: flextrain/checkpointing.py:1-418 - ``checkpointed_forward`` :259-287,
``checkpointed_backward`` :352-418 with its one-shot post-recomputation hook
:340-349, ``detach_variable`` :231-256, ``retrieve_tensor`` :290-310,
``retrieve_tensor_grads`` :313-337, ``CudaRNGStatesTracker`` and
``model_parallel_cuda_manual_seed`` :63-189.

A unit's forward runs under ``no_grad`` and keeps only its inputs and the RNG
state.  Backward restores the RNG state, recomputes the unit under
``enable_grad``, fires the hook (the engine uses it to start the previous
unit's gradient reduce-scatter so it overlaps the backward half rather than the
recompute), back-propagates and returns the input gradients.  Everything also
runs on CPU tensors; CUDA RNG state is touched only when CUDA is initialised.
"""
from __future__ import annotations

import contextlib
from dataclasses import dataclass
from typing import Any, Callable, Dict, Iterable, Optional, Tuple

import torch

_MODEL_PARALLEL_RNG_TRACKER_NAME = "model-parallel-rng"


def _cuda_active() -> bool:
    return torch.cuda.is_available() and torch.cuda.is_initialized()


def _set_cuda_rng_state(new_state: torch.Tensor, device: int = -1):
    """Install ``new_state`` on the current (or given) CUDA device."""
    if not _cuda_active():
        return
    if device == -1:
        device = torch.cuda.current_device()
    torch.cuda.set_rng_state(new_state, device)


class CudaRNGStatesTracker:
    """Named CUDA RNG streams.  ``fork(name)`` swaps the named state in, runs the
    body, stores the advanced state back and restores the ambient one."""

    def __init__(self):
        self.reset()

    def reset(self):
        self.states_: Dict[str, torch.Tensor] = {}
        self.seeds_ = set()

    def get_states(self) -> Dict[str, torch.Tensor]:
        return dict(self.states_)

    def set_states(self, states: Dict[str, torch.Tensor]):
        self.states_ = dict(states)

    def add(self, name: str, seed: int):
        if seed in self.seeds_:
            raise ValueError(f"seed {seed} already registered")
        if name in self.states_:
            raise ValueError(f"RNG state {name!r} already registered")
        self.seeds_.add(seed)
        if not torch.cuda.is_available():
            gen = torch.Generator()
            gen.manual_seed(seed)
            self.states_[name] = gen.get_state()
            return
        ambient = torch.cuda.get_rng_state()
        torch.cuda.manual_seed(seed)
        self.states_[name] = torch.cuda.get_rng_state()
        _set_cuda_rng_state(ambient)

    @contextlib.contextmanager
    def fork(self, name: str = _MODEL_PARALLEL_RNG_TRACKER_NAME):
        if name not in self.states_:
            raise KeyError(f"RNG state {name!r} was never added")
        if not _cuda_active():
            yield
            return
        ambient = torch.cuda.get_rng_state()
        _set_cuda_rng_state(self.states_[name])
        try:
            yield
        finally:
            self.states_[name] = torch.cuda.get_rng_state()
            _set_cuda_rng_state(ambient)


_CUDA_RNG_STATE_TRACKER = CudaRNGStatesTracker()


def get_cuda_rng_tracker() -> CudaRNGStatesTracker:
    return _CUDA_RNG_STATE_TRACKER


def model_parallel_cuda_manual_seed(seed: int):
    """Seed the default CUDA generator with ``seed`` (identical on every data
    parallel rank) and register a "model-parallel" stream at ``seed + 2718``.
    The engine is data-parallel only, so the tensor-parallel rank is 0."""
    tensor_parallel_rank = 0
    model_parallel_seed = seed + 2718 + tensor_parallel_rank
    _CUDA_RNG_STATE_TRACKER.reset()
    if torch.cuda.is_available():
        torch.cuda.manual_seed(seed)
    _CUDA_RNG_STATE_TRACKER.add(_MODEL_PARALLEL_RNG_TRACKER_NAME, model_parallel_seed)


class RNGStatePack:
    """CPU, CUDA and tracker RNG state at one instant."""

    def __init__(self, dummy: bool = False):
        self.dummy = dummy
        if dummy:
            return
        self.cpu_state = torch.get_rng_state()
        self.cuda_state = torch.cuda.get_rng_state() if _cuda_active() else None
        self.tracker_states = _CUDA_RNG_STATE_TRACKER.get_states()

    def recover_states(self):
        if self.dummy:
            return
        torch.set_rng_state(self.cpu_state)
        if self.cuda_state is not None:
            _set_cuda_rng_state(self.cuda_state)
        _CUDA_RNG_STATE_TRACKER.set_states(self.tracker_states)


@dataclass
class FWDContext:
    run_function: Callable
    fwd_rng_state: RNGStatePack
    fwd_args: Tuple


def detach_variable(inputs):
    """Detached copies (sharing storage) of every tensor in ``inputs``;
    floating tensors are marked ``requires_grad``.  A lone tensor comes back
    as a tensor, any other iterable as a tuple, anything else unchanged."""
    def one(x):
        if torch.is_tensor(x):
            x = x.detach()
            if x.is_floating_point() or x.is_complex():
                x.requires_grad_(True)
        return x

    if torch.is_tensor(inputs):
        return one(inputs)
    if not isinstance(inputs, Iterable):
        return inputs
    return tuple(one(x) for x in inputs)


def checkpointed_forward(run_function: Callable, *args, keep_rng: bool = True):
    """Run ``run_function(*args)`` without building a graph; return its output
    and the context ``checkpointed_backward`` needs to replay it."""
    ctx = FWDContext(run_function, RNGStatePack(dummy=not keep_rng), args)
    with torch.no_grad():
        outputs = run_function(*args)
    return outputs, ctx


def retrieve_tensor(values) -> torch.Tensor:
    """The single tensor of an inter-layer tuple (exactly one is allowed)."""
    if torch.is_tensor(values):
        return values
    found = [v for v in values if torch.is_tensor(v)]
    if len(found) != 1:
        raise ValueError(f"the passed-down tuple must hold exactly one tensor, found {len(found)}")
    return found[0]


def retrieve_tensor_grads(values):
    """Gradients of the tensors in ``values`` (``None`` for non-tensors)."""
    if torch.is_tensor(values):
        return values.grad
    return tuple(v.grad if torch.is_tensor(v) else None for v in values)


_POST_RECOMPUTATION: Optional[Callable[[], Any]] = None


def set_post_recomputation_function(fn: Optional[Callable[[], Any]]):
    """Arm a one-shot hook that fires between recompute and backward of the
    next ``checkpointed_backward`` call."""
    global _POST_RECOMPUTATION
    _POST_RECOMPUTATION = fn


def _fire_post_recomputation():
    global _POST_RECOMPUTATION
    fn, _POST_RECOMPUTATION = _POST_RECOMPUTATION, None
    if fn is not None:
        fn()


def checkpointed_backward(ctx: FWDContext, *grads):
    """Recompute the unit described by ``ctx`` and back-propagate ``grads``
    (one per output, ``None`` entries skipped).  Returns the gradients of
    ``ctx.fwd_args`` in order (``None`` for non-tensors or inputs that did not
    take part)."""
    inputs = detach_variable(ctx.fwd_args)
    resume = RNGStatePack(dummy=ctx.fwd_rng_state.dummy)
    ctx.fwd_rng_state.recover_states()
    with torch.enable_grad():
        outputs = ctx.run_function(*inputs)
    resume.recover_states()
    _fire_post_recomputation()

    if torch.is_tensor(outputs):
        outputs = (outputs,)
    pairs = [(o, g) for o, g in zip(outputs, grads)
             if torch.is_tensor(o) and o.requires_grad and g is not None]
    if pairs:
        torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
    return retrieve_tensor_grads(inputs)
