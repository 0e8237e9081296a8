"""Learning-rate schedules that drive ``optimizer.param_groups`` directly.

The reference's optimizer front-end is a plain object with ``param_groups``
(flextrain/optimizer.py:98-160), not a ``torch.optim.Optimizer``, so PyTorch's
schedulers refuse it; its users set ``group["lr"]`` themselves the way Megatron's
parameter scheduler does.  This is that piece: linear warm-up followed by cosine,
linear or no decay, evaluated per step from the step count alone (so a resumed run
only needs the count), applied to every group through its own base rate.

    sched = LRSchedule(opt, peak_lr=3e-4, warmup_steps=2000, total_steps=100000, decay="cosine")
    engine.register_post_step_function(sched.step)      # rate of step k+1 set after step k
"""
from __future__ import annotations

import math
from typing import Dict, Optional


class LRSchedule:
    def __init__(self, optimizer, peak_lr: Optional[float] = None, warmup_steps: int = 0,
                 total_steps: Optional[int] = None, decay: str = "cosine", min_lr_ratio: float = 0.1,
                 start_step: int = 0):
        if decay not in ("cosine", "linear", "constant"):
            raise ValueError("decay must be 'cosine', 'linear' or 'constant'")
        if decay != "constant" and (total_steps is None or total_steps <= warmup_steps):
            raise ValueError("a decaying schedule needs total_steps > warmup_steps")
        if warmup_steps < 0 or not 0.0 <= min_lr_ratio <= 1.0:
            raise ValueError("warmup_steps must be >= 0 and min_lr_ratio within [0, 1]")
        self.optimizer = optimizer
        self.warmup_steps, self.total_steps = warmup_steps, total_steps
        self.decay, self.min_lr_ratio = decay, min_lr_ratio
        # every group keeps its own peak: the given one, or the rate it was built with
        self.base_lrs = [float(peak_lr if peak_lr is not None else g["lr"]) for g in optimizer.param_groups]
        self.steps_done = start_step
        self._apply()

    def factor(self, step: int) -> float:
        """Multiplier of the peak rate for the update with index ``step`` (0-based)."""
        if self.warmup_steps and step < self.warmup_steps:
            return (step + 1) / self.warmup_steps
        if self.decay == "constant":
            return 1.0
        span = self.total_steps - self.warmup_steps
        t = min(max(step - self.warmup_steps, 0), span) / span
        shape = 0.5 * (1.0 + math.cos(math.pi * t)) if self.decay == "cosine" else 1.0 - t
        return self.min_lr_ratio + (1.0 - self.min_lr_ratio) * shape

    def _apply(self):
        f = self.factor(self.steps_done)
        for g, base in zip(self.optimizer.param_groups, self.base_lrs):
            g["lr"] = base * f

    def step(self):
        """Call once after every optimizer step (``register_post_step_function``)."""
        self.steps_done += 1
        self._apply()

    @property
    def current_lrs(self):
        return [g["lr"] for g in self.optimizer.param_groups]

    def state_dict(self) -> Dict[str, int]:
        return {"steps_done": self.steps_done}

    def load_state_dict(self, state: Dict[str, int]):
        self.steps_done = int(state["steps_done"])
        self._apply()
