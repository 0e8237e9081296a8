"""Failure detection on the host: heartbeats and failure notices in the process
group's key-value store, and a step watchdog.

The reference has nothing here beyond the process-group timeout
(flextrain/defaults.py:202-204): a rank that dies leaves the others hanging in a
collective for 30 minutes.  With this module every rank stamps a heartbeat per
step, posts a notice when it fails, and checks its peers before launching the
next step, so a failure is learnt on the host - never by faulting a GPU.  Waits
inside device kernels are bounded separately and report through error words
(``ft_gemm_error`` / ``ft_comm_error``).
"""
from __future__ import annotations

import threading
import time
from typing import Dict, Optional

import torch.distributed as tdist

from . import distributed as dist
from .logging import logger


class PeerFailure(RuntimeError):
    """Another rank reported a failure or stopped sending heartbeats."""


class FusedCollectiveTimeout(RuntimeError):
    """A rank waited longer than its limit for a peer inside a fused collective kernel; the
    kernels of that rank wrote nothing for the call in question, so the step it belongs to is
    incomplete.  Raised on every rank at the end of that step, after all ranks have switched
    to the library collectives."""


class Heartbeat:
    def __init__(self, prefix: str = "ft/health"):
        self.prefix = prefix
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        self._store = None
        if self.world > 1 and tdist.is_initialized():
            try:
                self._store = tdist.distributed_c10d._get_default_store()
            except Exception:
                self._store = None

    @property
    def active(self) -> bool:
        return self._store is not None

    def beat(self, step: int):
        if self._store is not None:
            self._store.set(f"{self.prefix}/beat/{self.rank}", f"{step}:{time.time():.3f}")

    def post_failure(self, message: str):
        if self._store is not None:
            try:
                self._store.set(f"{self.prefix}/failed/{self.rank}", message[:500])
                self._store.add(f"{self.prefix}/failures", 1)
            except Exception:
                pass

    def failures(self) -> Dict[int, str]:
        """Failure notices posted so far (rank -> message)."""
        if self._store is None:
            return {}
        try:
            if int(self._store.add(f"{self.prefix}/failures", 0)) == 0:
                return {}
        except Exception:
            return {}
        out = {}
        for r in range(self.world):
            key = f"{self.prefix}/failed/{r}"
            try:
                if self._store.check([key]):
                    out[r] = self._store.get(key).decode()
            except Exception:
                continue
        return out

    def check_peers(self, max_age: Optional[float] = None):
        """Raise ``PeerFailure`` if a peer posted a failure or (with ``max_age``)
        its last heartbeat is older than ``max_age`` seconds."""
        failed = {r: m for r, m in self.failures().items() if r != self.rank}
        if failed:
            raise PeerFailure("; ".join(f"rank {r} failed: {m}" for r, m in sorted(failed.items())))
        if max_age is None or self._store is None:
            return
        now = time.time()
        for r in range(self.world):
            if r == self.rank:
                continue
            key = f"{self.prefix}/beat/{r}"
            if not self._store.check([key]):
                continue
            stamp = float(self._store.get(key).decode().split(":")[1])
            if now - stamp > max_age:
                raise PeerFailure(f"rank {r} sent no heartbeat for {now - stamp:.1f} s")


class StepWatchdog:
    """Background thread that notices a training step running longer than
    ``limit`` seconds; it records the fact (and logs it) but kills nothing."""

    def __init__(self, limit: float):
        self.limit = float(limit)
        self.tripped = False
        self._start: Optional[float] = None
        self._stop = threading.Event()
        self._thread = None
        if self.limit > 0:
            self._thread = threading.Thread(target=self._run, name="ft-watchdog", daemon=True)
            self._thread.start()

    def step_started(self):
        self._start = time.monotonic()

    def step_finished(self):
        self._start = None

    def _run(self):
        while not self._stop.wait(min(1.0, max(self.limit / 4, 0.05))):
            start = self._start
            if start is not None and time.monotonic() - start > self.limit and not self.tripped:
                self.tripped = True
                logger.error(f"step watchdog: a training step has been running for more than "
                             f"{self.limit:.1f} s on rank {dist.get_rank()}")

    def reset(self):
        self.tripped = False

    def close(self):
        self._stop.set()
