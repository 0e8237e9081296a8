"""Greedy-snake order over (unit, micro_batch) tasks.

Parity: flextrain/scheduler.py:1-90.  One training step walks the task list
once: the first ``mb * (U-1)`` tasks are the forward pass over units
``0..U-2``; the remaining ``mb * U`` tasks are the backward pass, which starts
with the last unit (forward + loss + backward in one task) and descends to unit
0.  Inside a unit the micro-batches run ascending on even passes and
descending on odd ones, so the micro-batch that ends one unit starts the next
and its activation never leaves HBM.
"""
from dataclasses import dataclass
from typing import Iterator, List


@dataclass(frozen=True)
class LLMTask:
    is_forwarding: bool
    unit: int
    micro_batch: int


class GreedySnakeBlockScheduler:
    def __init__(self, micro_batch_count: int, unit_count: int):
        if micro_batch_count < 1 or unit_count < 1:
            raise ValueError("need at least one micro-batch and one unit")
        self.micro_batch_count = micro_batch_count
        self.unit_count = unit_count
        self._tasks: List[LLMTask] = self._build()
        self._num_fwd_task = micro_batch_count * (unit_count - 1)
        self._num_task = len(self._tasks)
        self._cursor = -1          # index of the task most recently handed out
        self._stop = self._num_task

    def _build(self) -> List[LLMTask]:
        mb, units = self.micro_batch_count, self.unit_count
        tasks: List[LLMTask] = []
        block = 0

        def sweep(unit, forwarding):
            nonlocal block
            order = range(mb) if block % 2 == 0 else range(mb - 1, -1, -1)
            tasks.extend(LLMTask(forwarding, unit, m) for m in order)
            block += 1

        for unit in range(units - 1):
            sweep(unit, True)
        for unit in range(units - 1, -1, -1):
            sweep(unit, False)
        return tasks

    # ------------------------------------------------------------ iteration
    def __iter__(self) -> Iterator[LLMTask]:
        """First call yields the forward tasks, second call the backward
        tasks, then the cycle repeats (the engine iterates twice per step)."""
        if self._cursor + 1 >= self._num_task:
            self._cursor = -1
        self._stop = self._num_fwd_task if self._cursor + 1 < self._num_fwd_task else self._num_task
        if self._cursor == -1 and self._num_fwd_task == 0:
            # a one-unit model has no forward-only tasks: first sweep is empty
            self._stop = 0 if not getattr(self, "_empty_fwd_done", False) else self._num_task
            self._empty_fwd_done = not getattr(self, "_empty_fwd_done", False)
        return self

    def __next__(self) -> LLMTask:
        if self._cursor + 1 >= self._stop:
            raise StopIteration
        self._cursor += 1
        return self._tasks[self._cursor]

    def reset(self):
        self._cursor = -1
        self._empty_fwd_done = False

    # ----------------------------------------------------------- properties
    @property
    def tasks(self) -> List[LLMTask]:
        return list(self._tasks)

    @property
    def forward_tasks(self) -> List[LLMTask]:
        return self._tasks[: self._num_fwd_task]

    @property
    def backward_tasks(self) -> List[LLMTask]:
        return self._tasks[self._num_fwd_task:]

    @property
    def curr_task(self) -> LLMTask:
        return self._tasks[max(self._cursor, 0)]

    @property
    def next_task(self) -> LLMTask:
        return self._tasks[(self._cursor + 1) % self._num_task]

    @property
    def last_task(self) -> LLMTask:
        return self._tasks[(self._cursor - 1) % self._num_task]

    @property
    def new_unit_entered(self) -> bool:
        return self._cursor % self.micro_batch_count == 0

    @property
    def in_first_unit(self) -> bool:
        return self.curr_task.unit == 0

    @property
    def in_last_unit(self) -> bool:
        return self.curr_task.unit == self.unit_count - 1

    @property
    def kth_micro_batch(self) -> int:
        """Position of the current task inside its unit sweep (0-based)."""
        return self._cursor % self.micro_batch_count
