"""Registry of the six user callbacks that split a model into pre / layers / post.

Parity: flextrain/llm_func.py:1-68.  The engine never receives a monolithic
``forward``; it drives these callbacks unit by unit and micro-batch by
micro-batch (flextrain/engine.py:116-258).

Contracts
---------
``get_batch() -> (pre_inputs, post_inputs, loss_inputs)``
    one micro-batch; called once per micro-batch at the first unit.
``pre_process(pre_inputs) -> (passed_down, every_layer)``
    ``passed_down`` is a tuple holding exactly one floating tensor (the
    inter-layer activation); ``every_layer`` is a (possibly empty) tuple of
    per-layer constants such as masks or RoPE tables.
``layer_forward(start, end)(*passed_down, *every_layer) -> passed_down``
    runs layers ``[start, end)``.
``post_process(passed_down, post_inputs) -> outputs`` and
``loss(outputs, loss_inputs)`` -> a scalar tensor or an iterable whose first
    one-element tensor is the loss.
``get_layer(i)`` is kept for API parity; the engine does not call it.
"""
from typing import Any, Callable, Iterable, Sequence, Tuple

from torch import Tensor
from torch.nn import Module


def _unset(name):
    def missing(*_a, **_k):
        raise NotImplementedError(f"LLMFunc.{name} is not registered: call set_llm_func(...) first")
    return staticmethod(missing)


class LLMFunc:
    get_layer = _unset("get_layer")
    get_batch = _unset("get_batch")
    pre_process = _unset("pre_process")
    layer_forward = _unset("layer_forward")
    post_process = _unset("post_process")
    loss = _unset("loss")


def set_llm_func(get_layer: Callable[[int], Module],
                 get_batch: Callable[[], Tuple[Tuple, Tuple, Tuple]],
                 pre_process: Callable[[Tuple], Tuple[Tuple, Tuple]],
                 layer_forward: Callable[[int, int], Callable[..., Tuple]],
                 post_process: Callable[[Tuple, Tuple], Tuple],
                 loss: Callable[[Tuple, Tuple], Sequence[Any]]):
    LLMFunc.get_layer = staticmethod(get_layer)
    LLMFunc.get_batch = staticmethod(get_batch)
    LLMFunc.pre_process = staticmethod(pre_process)
    LLMFunc.layer_forward = staticmethod(layer_forward)
    LLMFunc.post_process = staticmethod(post_process)
    LLMFunc.loss = staticmethod(loss)


def reset_llm_func():
    """Forget the registered callbacks (and with them the model they close over)."""
    for name in ("get_layer", "get_batch", "pre_process", "layer_forward", "post_process", "loss"):
        setattr(LLMFunc, name, _unset(name))


def retrieve_llm_loss(loss_rsts) -> Tensor:
    """The numerical loss inside whatever the user's loss callback returned."""
    if isinstance(loss_rsts, Tensor):
        if loss_rsts.numel() != 1:
            raise ValueError("the loss tensor must hold exactly one element")
        return loss_rsts
    if isinstance(loss_rsts, Iterable):
        for item in loss_rsts:
            if isinstance(item, Tensor) and item.numel() == 1:
                return item
    raise ValueError("no one-element tensor found in the return value of the loss callback")
