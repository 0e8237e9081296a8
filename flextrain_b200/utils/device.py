"""Streams and events that work the same on ``cuda`` and on ``cpu``.

The engine orders its copy / collective / compute work with events between a
few dedicated streams (never with a device-wide synchronise per micro-batch,
unlike flextrain/memory/__init__.py:394-395).  On the CPU backend every
operation is synchronous, so streams and events degenerate to no-ops and the
same engine code runs under gloo in tests.
"""
from __future__ import annotations

import contextlib
from typing import Optional

import torch

from . import distributed as dist


class Event:
    """A point in a stream's work queue.  ``None`` inside means "already done"."""

    __slots__ = ("_ev",)

    def __init__(self, ev: Optional["torch.cuda.Event"] = None):
        self._ev = ev

    def wait(self, stream: Optional["Stream"] = None):
        """Make ``stream`` (default: the current stream) wait for this point."""
        if self._ev is None:
            return
        if stream is None or stream.raw is None:
            torch.cuda.current_stream().wait_event(self._ev)
        else:
            stream.raw.wait_event(self._ev)

    def synchronize(self):
        if self._ev is not None:
            self._ev.synchronize()

    def query(self) -> bool:
        return True if self._ev is None else self._ev.query()


DONE = Event(None)


class Stream:
    """A CUDA stream, or a stand-in on CPU (``raw is None``)."""

    def __init__(self, name: str, cuda: bool, priority: int = 0, current: bool = False):
        self.name = name
        if not cuda:
            self.raw = None
        elif current:
            self.raw = torch.cuda.current_stream()
        else:
            self.raw = torch.cuda.Stream(priority=priority)

    @contextlib.contextmanager
    def use(self):
        if self.raw is None:
            yield self
        else:
            with torch.cuda.stream(self.raw):
                yield self

    def record(self) -> Event:
        if self.raw is None:
            return DONE
        ev = torch.cuda.Event()
        ev.record(self.raw)
        return ev_wrap(ev)

    def wait(self, event: Optional[Event]):
        if event is not None:
            event.wait(self)

    def wait_stream(self, other: "Stream"):
        if self.raw is not None and other.raw is not None:
            self.raw.wait_stream(other.raw)

    def synchronize(self):
        if self.raw is not None:
            self.raw.synchronize()

    @property
    def handle(self) -> int:
        return 0 if self.raw is None else self.raw.cuda_stream


def ev_wrap(ev) -> Event:
    return Event(ev)


class StreamSet:
    """The streams one rank uses: the compute stream (PyTorch's current
    stream), one for host->device + gather traffic, one for device->host +
    reduce traffic and one for optimizer kernels."""

    def __init__(self, device: Optional[torch.device] = None):
        device = device or dist.current_device()
        self.device = device
        self.cuda = device.type == "cuda"
        self.compute = Stream("compute", self.cuda, current=True)
        self.h2d = Stream("h2d", self.cuda, priority=-1)
        self.d2h = Stream("d2h", self.cuda, priority=-1)
        self.opt = Stream("opt", self.cuda)

    def synchronize(self):
        if self.cuda:
            torch.cuda.synchronize(self.device)


_STREAMS: Optional[StreamSet] = None


def get_streams() -> StreamSet:
    global _STREAMS
    if _STREAMS is None or _STREAMS.device != dist.current_device():
        _STREAMS = StreamSet()
    return _STREAMS


def reset_streams():
    global _STREAMS
    _STREAMS = None
