"""Inter-layer coordinator: tiering of the activation checkpoint of every
``(unit, micro_batch)`` and of the activation gradient handed from unit to unit
in backward.

Parity: flextrain/memory/coordinator/interlayer.py:1-373 (lazy init on first
offload :41-147, landing buffers :79-93, NVMe margin :108-113, prefetch /
offload bodies :203-231,280-294, hooks :252-360).

Each tensor is cut ``[HBM | pinned DRAM | NVMe]`` by ``split_ratio.checkpoint``
(checkpoints) or ``[HBM | DRAM]`` by ``split_ratio.gradient`` (activation
gradients).  ``put`` copies the non-HBM pieces out on the d2h stream behind a
compute event and drops the producer's tensor once that is done; ``prefetch``
re-assembles a tensor into one of two HBM landing buffers on the h2d stream one
task ahead of its consumer; ``get`` makes the compute stream wait for it.  With
an HBM share of 1.0 the store keeps the tensor itself and nothing is copied -
the normal case on a 180 GB part.  The NVMe piece of a checkpoint is the file
``rank{r}_CKPT_layer{u}.mb{j}.swp``; the first and last micro-batch of every
unit (the snake turn) never go to NVMe.

NVMe pieces never make the Python thread wait for a disk or a copy: a worker thread
per store writes a piece once its device-to-host copy has landed in a staging buffer,
and on the way back reads it into another staging buffer and itself queues the
host-to-device copies that assemble the landing buffer.  The consumer only waits (on
the host) for that queueing to have happened and (on the compute stream) for the event
recorded behind it.
"""
from __future__ import annotations

import queue
import threading
from concurrent.futures import Future
from dataclasses import dataclass
from typing import Dict, Hashable, Optional, Tuple

import torch

from ...config import get_flextrain_config
from ...utils import distributed as dist
from ...utils.device import DONE, Event, get_streams
from .. import (tier_copy, FlexTrainDataID, FlexTrainDataType, allocate_memory, get_split_numels)
from ..nvme_swapper import get_nvme_swapper
from ...scheduler import LLMTask


@dataclass(frozen=True)
class InterLayerTask(LLMTask):
    """A scheduler task together with the inter-unit tensor it carries
    (flextrain/memory/coordinator/interlayer.py:27-28).  The stores below are keyed by
    ``(unit, micro_batch)`` directly; the class is kept for code that builds such tasks."""
    tensor: Optional[torch.Tensor] = None



class _DiskWorker:
    """One thread that runs the NVMe transfers of a store in the order they were queued."""

    def __init__(self, device):
        self._q: "queue.Queue" = queue.Queue()
        self._device = device
        self._thread = threading.Thread(target=self._run, name="ft-ckpt-nvme", daemon=True)
        self._thread.start()

    def submit(self, fn) -> Future:
        fut: Future = Future()
        self._q.put((fn, fut))
        return fut

    def _run(self):
        if self._device.type == "cuda":
            torch.cuda.set_device(self._device)
        while True:
            fn, fut = self._q.get()
            if fn is None:
                fut.set_result(None)
                return
            try:
                fut.set_result(fn())
            except BaseException as exc:          # surfaced by whoever waits on the future
                fut.set_exception(exc)

    def shutdown(self):
        fut: Future = Future()
        self._q.put((None, fut))
        fut.result()


class _Slot:
    __slots__ = ("shape", "dtype", "whole", "hot", "gpu", "cpu", "nvme_id", "stored", "landing",
                 "ready", "io", "ready_future")

    def __init__(self):
        self.whole = None      # the tensor itself when everything stays in HBM
        self.hot = None        # the producer's tensor, kept for an immediate consumer
        self.gpu = None
        self.cpu = None
        self.nvme_id = None
        self.stored: Event = DONE
        self.landing = None
        self.ready: Optional[Event] = None
        self.io = None              # Future of the NVMe write of this slot's piece
        self.ready_future = None    # Future -> Event: the worker queued the copies into the landing buffer


class TieredTensorStore:
    """Keyed store of equally sized tensors with a fixed tier split."""

    def __init__(self, data_type: FlexTrainDataType, ratios: Tuple[float, float], allow_nvme: bool):
        self.data_type = data_type
        self.ratios = ratios
        self.allow_nvme = allow_nvme
        self.device = dist.current_device()
        self.streams = get_streams()
        self._slots: Dict[Hashable, _Slot] = {}
        self._numel = None
        self._tiers = None
        self._landing = []
        self._landing_free = []
        self._nvme_stage = []
        self._pool_cpu = []             # recycled pinned pieces
        self._pool_cpu_wide = []        # pinned buffers of DRAM + NVMe share (margin micro-batches)
        self._pool_gpu = []
        self._worker: Optional[_DiskWorker] = None
        self.bytes_d2h = 0
        self.bytes_h2d = 0

    # ----------------------------------------------------------------- init
    def _lazy_init(self, t: torch.Tensor):
        self._numel = t.numel()
        self._dtype = t.dtype
        itemsize = t.element_size()
        gpu, cpu = self.ratios
        if not self.allow_nvme:
            cpu = 1.0 - gpu
        self._tiers = get_split_numels(self._numel, (gpu, cpu), itemsize)
        self.all_hbm = self._tiers[1] == 0 and self._tiers[2] == 0
        if not self.all_hbm:
            self._landing = [allocate_memory(self._numel, t.dtype, self.device) for _ in range(2)]
            self._landing_free = [DONE, DONE]
            if self._tiers[2]:
                # two staging buffers per direction: a piece on its way out never waits for one coming in
                self._out_stage = [allocate_memory(self._tiers[2], t.dtype, "cpu", True) for _ in range(2)]
                self._in_stage = [allocate_memory(self._tiers[2], t.dtype, "cpu", True) for _ in range(2)]
                for stage in self._out_stage + self._in_stage:
                    get_nvme_swapper().register_staging(stage)
                self._out_busy = [None, None]          # Future of the write that last used the buffer
                self._in_copied = [DONE, DONE]         # event: the last copy out of the buffer has run
                self._out_next = self._in_next = 0
                self._worker = _DiskWorker(self.device)

    def _data_id(self, key):
        if isinstance(key, tuple):                  # (unit, micro-batch)
            return FlexTrainDataID(self.data_type, key[0], micro_batch=key[1])
        return FlexTrainDataID(self.data_type, "all", micro_batch=key)

    # ------------------------------------------------------------------ put
    @torch.no_grad()
    def put(self, key, tensor: torch.Tensor, pin_to_dram: bool = False, hot: bool = False,
            store: bool = True):
        """Store ``tensor`` (produced on the compute stream).  ``pin_to_dram``
        keeps the would-be NVMe piece in DRAM (margin micro-batches).  ``hot``
        keeps the tensor itself for the very next consumer (the snake turn);
        ``store=False`` then skips the tier copies because nobody else will
        ever ask for it."""
        if self._numel is None:
            self._lazy_init(tensor)
        if tensor.numel() != self._numel:
            raise ValueError("all tensors of one store must have the same size")
        slot = self._slots.get(key) or _Slot()
        self._slots[key] = slot
        slot.shape, slot.dtype = tensor.shape, tensor.dtype
        self._settle(slot)
        if slot.landing is not None:
            self._landing_free[slot.landing] = self.streams.compute.record()
        slot.ready, slot.landing = None, None
        slot.hot = tensor if hot else None
        if self.all_hbm:
            slot.whole = tensor
            return
        if hot and not store:
            return
        g, c, n = self._tiers
        flat = tensor.reshape(-1)
        produced = self.streams.compute.record()
        st = self.streams
        with st.d2h.use():
            st.d2h.wait(produced)
            if g:
                slot.gpu = slot.gpu if slot.gpu is not None else (
                    self._pool_gpu.pop() if self._pool_gpu else
                    allocate_memory(g, tensor.dtype, self.device))
                tier_copy(slot.gpu, flat[:g])
            host_n = c + (n if (pin_to_dram or not n) else 0)
            if pin_to_dram and n:
                # whole non-HBM part stays in DRAM
                if slot.cpu is None or slot.cpu.numel() != c + n:
                    # margin micro-batches come back every step: their wide buffers are pooled too
                    slot.cpu = self._pool_cpu_wide.pop() if self._pool_cpu_wide else \
                        allocate_memory(c + n, tensor.dtype, "cpu", True)
                tier_copy(slot.cpu, flat[g:])
                slot.nvme_id = None
            else:
                if c:
                    if slot.cpu is None or slot.cpu.numel() != c:
                        slot.cpu = self._pool_cpu.pop() if self._pool_cpu else \
                            allocate_memory(c, tensor.dtype, "cpu", True)
                    tier_copy(slot.cpu, flat[g:g + c])
                if n:
                    i = self._out_next
                    self._out_next = (i + 1) % 2
                    if self._out_busy[i] is not None:
                        self._out_busy[i].result()        # the write two pieces back still owns the buffer
                    stage = self._out_stage[i]
                    tier_copy(stage, flat[g + c:])
                    copied = st.d2h.record()
                    nvme_id = self._data_id(key)
                    slot.nvme_id = nvme_id

                    def write(copied=copied, stage=stage, nvme_id=nvme_id):
                        copied.synchronize()
                        get_nvme_swapper().swap_out(nvme_id, stage)

                    slot.io = self._worker.submit(write)
                    self._out_busy[i] = slot.io
            self.bytes_d2h += (self._numel - g) * tensor.element_size()
            slot.stored = st.d2h.record()
        # the producer's storage may be recycled only after the copies have read it
        if tensor.is_cuda:
            tensor.record_stream(st.d2h.raw)

    # ------------------------------------------------------------- prefetch
    @torch.no_grad()
    def prefetch(self, key):
        """Start re-assembling ``key`` into a landing buffer (h2d stream)."""
        slot = self._slots.get(key)
        if slot is None or self.all_hbm or slot.ready is not None or slot.ready_future is not None \
                or slot.hot is not None:
            return
        g, c, n = self._tiers
        idx = 0 if self._landing_free[0] is not None else 1
        if self._landing_free[idx] is None:
            raise RuntimeError("both landing buffers are in use: consume one before prefetching")
        free_ev = self._landing_free[idx]
        self._landing_free[idx] = None
        land = self._landing[idx]
        st = self.streams
        slot.landing = idx
        if slot.nvme_id is None:
            slot.ready = self._assemble(slot, land, free_ev, None, None)
            return
        # the NVMe piece comes back on the worker thread, which then queues every copy into the
        # landing buffer itself; the Python thread goes on
        i = self._in_next
        self._in_next = (i + 1) % 2
        stage, written = self._in_stage[i], slot.io

        def read(i=i, stage=stage, written=written, nvme_id=slot.nvme_id):
            if written is not None:
                written.result()                       # the piece is on disk
            self._in_copied[i].synchronize()            # the previous piece has left the buffer
            get_nvme_swapper().swap_in(nvme_id, stage)
            ready = self._assemble(slot, land, free_ev, stage, i)
            return ready

        slot.ready_future = self._worker.submit(read)
        slot.io = None

    def _assemble(self, slot, land, free_ev, stage, stage_index) -> Event:
        """Queue the copies that put a tensor together in its landing buffer (h2d stream)."""
        g, c, n = self._tiers
        st = self.streams
        with st.h2d.use():
            st.h2d.wait(free_ev)
            st.h2d.wait(slot.stored)
            if g:
                tier_copy(land[:g], slot.gpu)
            if slot.cpu is not None:
                tier_copy(land[g:g + slot.cpu.numel()], slot.cpu)
            if stage is not None:
                tier_copy(land[g + c:], stage)
            self.bytes_h2d += (self._numel - g) * land.element_size()
            ready = st.h2d.record()
        if stage is not None:
            self._in_copied[stage_index] = ready
        return ready

    # ------------------------------------------------------------------ get
    def get(self, key) -> torch.Tensor:
        """The tensor on the device, valid on the compute stream."""
        slot = self._slots[key]
        if self.all_hbm:
            return slot.whole
        if slot.hot is not None:
            hot, slot.hot = slot.hot, None
            return hot
        if slot.ready is None and slot.ready_future is None:
            self.prefetch(key)
        if slot.ready_future is not None:
            slot.ready, slot.ready_future = slot.ready_future.result(), None
        self.streams.compute.wait(slot.ready)
        return self._landing[slot.landing].view(slot.shape)

    @staticmethod
    def _settle(slot):
        """A read-back that was started and never consumed must have queued its copies before
        the landing buffer changes hands."""
        if slot.ready_future is not None:
            fut, slot.ready_future = slot.ready_future, None
            slot.ready = fut.result()

    def done_with(self, key, drop: bool = False):
        """The consumer has queued its last read of ``key`` on the compute stream."""
        slot = self._slots.get(key)
        if slot is None:
            return
        self._settle(slot)
        if slot.landing is not None:
            self._landing_free[slot.landing] = self.streams.compute.record()
            slot.landing, slot.ready = None, None
        if drop:
            self.drop(key)

    def drop(self, key):
        slot = self._slots.pop(key, None)
        if slot is None:
            return
        self._settle(slot)
        if slot.landing is not None:
            self._landing_free[slot.landing] = self.streams.compute.record()
        if slot.cpu is not None and self._tiers and slot.cpu.numel() == self._tiers[1]:
            self._pool_cpu.append(slot.cpu)
        elif slot.cpu is not None and self._tiers and self._tiers[2] and \
                slot.cpu.numel() == self._tiers[1] + self._tiers[2]:
            self._pool_cpu_wide.append(slot.cpu)
        if slot.gpu is not None:
            self._pool_gpu.append(slot.gpu)
        if slot.nvme_id is not None and slot.io is not None:
            slot.io.result()

    def __contains__(self, key):
        return key in self._slots

    def clear(self):
        for key in list(self._slots):
            self.drop(key)

    def close(self):
        """Stop the worker thread (after what it still holds has run)."""
        if self._worker is not None:
            self._worker.shutdown()
            self._worker = None


class FlexTrainInterLayerCoordinator:
    """Two stores: activation checkpoints keyed ``(unit, micro_batch)`` and
    activation gradients keyed ``micro_batch``."""

    def __init__(self):
        cfg = get_flextrain_config()
        self.ckpt = TieredTensorStore(FlexTrainDataType.CKPT, cfg.split_ratio.checkpoint, True)
        self.grad = TieredTensorStore(FlexTrainDataType.GRAD, cfg.split_ratio.gradient, False)

    def traffic(self):
        return {"ckpt_d2h": self.ckpt.bytes_d2h, "ckpt_h2d": self.ckpt.bytes_h2d,
                "grad_d2h": self.grad.bytes_d2h, "grad_h2d": self.grad.bytes_h2d}


_INTER: Optional[FlexTrainInterLayerCoordinator] = None


def get_interlayer_coordinator() -> FlexTrainInterLayerCoordinator:
    global _INTER
    if _INTER is None:
        _INTER = FlexTrainInterLayerCoordinator()
    return _INTER


def reset_interlayer_coordinator():
    global _INTER
    if _INTER is not None:
        _INTER.ckpt.close()
        _INTER.grad.close()
    _INTER = None
