"""Per-step metrics sink.

The reference reports nothing while it trains (no throughput counters, no metrics file:
its only timers live inside flextrain/auto_config.py:100-164).  ``MetricsLog`` appends one
JSON object per optimizer step to a file (rank 0 only unless told otherwise):

    step, time, loss, step_seconds, tokens_per_s, tflops_per_gpu, loss_scale, grad_norm,
    skipped_steps, lr, traffic_bytes{h2d, d2h, nvme_read, nvme_write, gather, reduce, ...}

and can expose the same numbers as Prometheus gauges (``prometheus_client``, optional).

    log = MetricsLog("metrics.jsonl", engine, tokens_per_step=B * S, flops_per_token=f, n_gpus=W)
    for _ in range(steps):
        losses = engine.train_iteration()
        log.step(losses)
"""
from __future__ import annotations

import json
import time
from typing import Any, Dict, Iterable, Optional

from . import distributed as dist


def _loss_value(losses) -> Optional[float]:
    """Mean of the per-micro-batch loss results (tensors, floats, or tuples whose first
    one-element tensor is the loss, as the ``loss`` callback may return them)."""
    if losses is None:
        return None
    vals = []
    for item in (losses if isinstance(losses, (list, tuple)) else [losses]):
        if isinstance(item, (list, tuple)):
            item = next((x for x in item if hasattr(x, "numel") and x.numel() == 1), None)
        if item is None:
            continue
        vals.append(float(item.detach()) if hasattr(item, "detach") else float(item))
    return sum(vals) / len(vals) if vals else None


class MetricsLog:
    def __init__(self, path: Optional[str], engine, tokens_per_step: int = 0, flops_per_token: float = 0.0,
                 n_gpus: Optional[int] = None, all_ranks: bool = False, prometheus_port: Optional[int] = None,
                 extra: Optional[Dict[str, Any]] = None):
        self.engine = engine
        self.tokens_per_step = int(tokens_per_step)
        self.flops_per_token = float(flops_per_token)
        self.n_gpus = int(n_gpus if n_gpus is not None else max(1, dist.get_world_size()))
        self.extra = dict(extra or {})
        self.active = all_ranks or dist.get_rank() == 0
        self._file = open(path, "a", buffering=1) if (path and self.active) else None
        self._last_wall = time.perf_counter()
        self._gauges = None
        if prometheus_port is not None and self.active:
            self._start_prometheus(int(prometheus_port))

    # ------------------------------------------------------------------ record
    def step(self, losses=None, **fields) -> Dict[str, Any]:
        """Record the step that just finished; returns the record (on every rank)."""
        now = time.perf_counter()
        eng = self.engine
        seconds = now - self._last_wall              # wall time between two calls: includes data loading
        self._last_wall = now
        rec: Dict[str, Any] = {"step": int(eng.global_steps), "time": time.time(),
                               "loss": _loss_value(losses), "step_seconds": seconds}
        if self.tokens_per_step and seconds > 0:
            tps = self.tokens_per_step / seconds
            rec["tokens_per_s"] = tps
            if self.flops_per_token:
                rec["tflops_per_gpu"] = tps * self.flops_per_token / self.n_gpus / 1e12
        rec["loss_scale"] = float(eng.loss_scale)
        rec["skipped_steps"] = int(eng.skipped_steps)
        norm = getattr(eng.opts, "last_grad_norm", None)
        if norm is not None:
            rec["grad_norm"] = float(norm)
        try:
            rec["lr"] = float(eng.optimizer.param_groups[0]["lr"])
        except (AttributeError, KeyError, IndexError):
            pass
        rec["traffic_bytes"] = eng.stats(reset=True)["traffic_bytes"]
        rec.update(self.extra)
        rec.update(fields)
        if self._file is not None:
            self._file.write(json.dumps(rec) + "\n")
        if self._gauges is not None:
            self._publish(rec)
        return rec

    def close(self):
        if self._file is not None:
            self._file.close()
            self._file = None

    # -------------------------------------------------------------- prometheus
    def _start_prometheus(self, port: int):
        from prometheus_client import CollectorRegistry, Gauge, start_http_server
        self.registry = CollectorRegistry()
        names = ("step", "loss", "step_seconds", "tokens_per_s", "tflops_per_gpu", "loss_scale", "grad_norm",
                 "skipped_steps", "lr")
        self._gauges = {n: Gauge(f"flextrain_{n}", f"flextrain {n}", registry=self.registry) for n in names}
        self._traffic = Gauge("flextrain_traffic_bytes", "bytes moved in the last step", ["kind"],
                              registry=self.registry)
        if port > 0:
            start_http_server(port, addr="127.0.0.1", registry=self.registry)

    def _publish(self, rec: Dict[str, Any]):
        for name, gauge in self._gauges.items():
            v = rec.get(name)
            if v is not None:
                gauge.set(v)
        for kind, nbytes in rec.get("traffic_bytes", {}).items():
            self._traffic.labels(kind=kind).set(nbytes)


def read_metrics(path: str) -> Iterable[Dict[str, Any]]:
    with open(path) as f:
        return [json.loads(line) for line in f if line.strip()]
