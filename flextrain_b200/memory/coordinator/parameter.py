"""Parameter coordinator: ZeRO-3 partition, tiering and one-unit-ahead gather of
the layer parameters.

Parity: flextrain/memory/coordinator/parameter.py:1-684 (geometry :96-165,
buffers :71-91, ``init_unit_parameters`` :274-352, NVMe load/offload :383-446,
gather task :470-519, hooks :521-642, warm-up/clear :644-671).

Geometry (deliberately simpler than the reference's micro-batch x rank
interleave, and with a real HBM tier)
  * a unit = ``checkpoint_interval`` consecutive layers, flattened in device
    dtype and padded to ``aligned_unit_numel`` (a multiple of
    ``world * 4096 / itemsize``);
  * rank ``r`` owns the contiguous shard ``[r*S, (r+1)*S)``, ``S = aligned / world``;
  * the shard is cut ``[HBM | pinned DRAM | NVMe]`` by ``split_ratio.parameter``
    at page-aligned points; the NVMe piece of unit ``u`` is the file
    ``rank{r}_PARA_layer{u}.swp``.

Working set in HBM: ``num_unit_buffers`` full-unit buffers forming a ring.
``submit_gather(u)`` assembles the local shard into the next free buffer on the
h2d stream (D2D + H2D copies), all-gathers it in place and records an event;
``acquire(u)`` makes the compute stream wait for that event and points the
unit's ``nn.Parameter``s at the buffer; ``release(u)`` returns the buffer to
the ring behind a compute-stream event.  No device-wide synchronisation is
involved.
"""
from __future__ import annotations

from collections import deque
from typing import Dict, List, Optional, Sequence

import torch

from ...config import get_flextrain_config
from ...defaults import PAGE_SIZE
from ...utils import distributed as dist
from ...utils.device import DONE, Event, get_streams
from ...utils.logging import rank0_logger
from .. import (tier_copy, ContiguousParaGroup, FlexTrainDataID, FlexTrainDataType, Waitable,
                allocate_memory, get_split_numels, partition_aligned_numel)
from ..nvme_swapper import get_nvme_swapper


class _PendingFirstGemm:
    """Marker on a parameter whose rows are not all in the gathered buffer yet: the first
    ``linear`` that uses the parameter runs the all-gather GEMM, which completes the buffer."""

    def __init__(self, coordinator, unit: int, idx: int):
        self.coordinator, self.unit, self.idx = coordinator, unit, idx

    def covers(self, rows: int, cols: int) -> bool:
        from ...parallel import fused
        return fused.ag_gemm_covers(rows, cols, 0, fused.AG_GEMM_CHUNK)

    def run(self, x2: torch.Tensor, out: torch.Tensor):
        c = self.coordinator
        c._run_first_gemm(self.unit, self.idx, x2, out)
        c._first_gemm_pending.pop(self.idx, None)
        c._first_gemm[self.unit][0]._ft_gather = None

    def complete_without_product(self):
        """Bring the matrix in with a plain range gather (a product the fused kernel does not
        cover, e.g. fewer than 129 rows)."""
        c = self.coordinator
        from ...parallel import fused
        _p, w_lo, rows, cols = c._first_gemm[self.unit]
        page = c._flag_page
        fused.peer_gather_range(c.world, c.rank, c._symm[self.idx].ptr_array(), page.ptr_array(),
                                page.next_seq("gather"), c.shard_numel * c.itemsize, w_lo,
                                w_lo + rows * cols * c.itemsize, num_copiers=c._cfg.engine.fused_blocks)
        c._first_gemm_pending.pop(self.idx, None)
        c._first_gemm[self.unit][0]._ft_gather = None


class FlexTrainParaCoordinator:
    def __init__(self):
        self._initialized = False
        self.num_layers = 0
        self.num_units = 0
        self._unit_groups: Dict[int, ContiguousParaGroup] = {}
        self._unit_layers: Dict[int, List[torch.nn.Module]] = {}

    # ------------------------------------------------------------ geometry
    @property
    def is_initialized(self):
        return self._initialized

    def _init_coordinator(self, num_layers: int, first_unit_numel: int):
        cfg = get_flextrain_config()
        self._cfg = cfg
        self.device = dist.current_device()
        self.streams = get_streams()
        self.world = dist.get_world_size()
        self.rank = dist.get_rank()
        self.device_dtype = cfg.mixed_precision.device_dtype
        self.itemsize = torch.empty((), dtype=self.device_dtype).element_size()
        self.num_layers = num_layers
        self.checkpoint_interval = cfg.checkpoint_interval
        self.num_units = (num_layers - 1) // cfg.checkpoint_interval + 1
        self.unit_numel = first_unit_numel
        # one rank's shard is a multiple of the page (O_DIRECT pieces) and, on several ranks, of the
        # 8 KiB ownership granule of the all-gather GEMM
        page = 8192 if self.world > 1 else PAGE_SIZE
        self.aligned_unit_numel = partition_aligned_numel(first_unit_numel, self.world, self.itemsize, page)
        self.shard_numel = self.aligned_unit_numel // self.world
        self.tier_numels = get_split_numels(self.shard_numel, cfg.split_ratio.parameter, self.itemsize)
        g, c, n = self.tier_numels
        self.num_buffers = cfg.engine.num_unit_buffers
        # with the fused collectives the ring buffers are peer-mapped: every rank pulls
        # the other ranks' shards straight out of their ring buffers (no NCCL all-gather)
        self._peer_gather = self._want_peer_gather(cfg)
        self._symm = []
        if self._peer_gather:
            from ...parallel.symm_mem import SymmetricBuffer, get_flag_page
            self._flag_page = get_flag_page()
            self._symm = [SymmetricBuffer(self.aligned_unit_numel * self.itemsize)
                          for _ in range(self.num_buffers)]
            self._buffers = [sb.tensor(self.device_dtype) for sb in self._symm]
        else:
            self._buffers = [allocate_memory(self.aligned_unit_numel, self.device_dtype, self.device)
                             for _ in range(self.num_buffers)]
        self._free = deque((i, DONE) for i in range(self.num_buffers))
        self._inflight: Dict[int, tuple] = {}      # unit -> (buffer index, ready event)
        self._held: Dict[int, int] = {}            # unit -> buffer index (linked)
        self._cached: Dict[int, tuple] = {}        # unit -> (buffer index, free event), still valid
        self._version: Dict[int, int] = {}         # bumped whenever a unit's shard changes
        self._held_version: Dict[int, int] = {}
        # a rank that holds whole units in HBM can compute straight from the base copy
        self._direct = self.world == 1 and c == 0 and n == 0
        self._gpu_base: Dict[int, torch.Tensor] = {}
        self._cpu_base: Dict[int, torch.Tensor] = {}
        self._gpu_base_ready: Dict[int, Event] = {}   # last device-side write to gpu_base[u]
        self._host_ready: Dict[int, List[Waitable]] = {}  # host-side updates still running
        self._nvme_landing = [allocate_memory(n, self.device_dtype, "cpu", True) for _ in range(2)] \
            if n else []
        for landing in self._nvme_landing:
            get_nvme_swapper().register_staging(landing)
        self._nvme_loads: Dict[int, tuple] = {}    # unit -> (landing index, read handle)
        self._landing_busy = [DONE for _ in self._nvme_landing]
        self._nvme_next = 0
        # The matrix a unit's forward multiplies first can be left out of the unit gather and
        # brought in by the all-gather GEMM itself (``ops.cuda_ops.linear`` sees the marker that
        # ``acquire`` puts on the parameter): unit -> (parameter, byte offset, rows, columns)
        self._first_gemm: Dict[int, tuple] = {}
        self._first_gemm_pending: Dict[int, int] = {}      # buffer index -> unit still without it
        self._first_gemm_on = self._peer_gather and cfg.engine.fused_first_gemm is not False
        self.first_gemm_calls = 0
        self._initialized = True
        rank0_logger.info(
            f"parameter geometry: units={self.num_units} unit_numel={self.unit_numel} "
            f"aligned={self.aligned_unit_numel} shard={self.shard_numel} "
            f"tiers(HBM,DRAM,NVMe)={self.tier_numels} dtype={self.device_dtype}")

    def _want_peer_gather(self, cfg) -> bool:
        want = cfg.engine.fused_collectives
        if want is False or self.device.type != "cuda" or self.world == 1 or self.world > 8:
            return False
        from ...parallel.symm_mem import peer_access_available
        ok = peer_access_available()
        if want is True and not ok:
            raise RuntimeError("engine.fused_collectives=true needs peer access between all ranks")
        return bool(ok)

    def _note_first_gemm(self, unit: int, layers, group: ContiguousParaGroup):
        """A layer class may name, in ``ft_first_gemm_weight``, the 2-D parameter its forward
        multiplies first.  When the placement suits the fused kernel the unit gather leaves that
        matrix out and the first product of the unit brings it in."""
        if not self._first_gemm_on or not layers:
            return
        name = getattr(layers[0], "ft_first_gemm_weight", None)
        w = getattr(layers[0], name, None) if name else None
        if w is None:
            return
        from ...parallel import fused
        for p, off, shape in zip(group.paras, group.offsets, group.shapes):
            if p is w and len(shape) == 2 and self.itemsize == 2:
                shard_bytes = self.shard_numel * self.itemsize
                if fused.ag_gemm_covers(1 << 20, shape[1], off * self.itemsize, shard_bytes):
                    self._first_gemm[unit] = (p, off * self.itemsize, shape[0], shape[1])
                return

    def fused_first_gemm_state(self) -> str:
        if not getattr(self, "_first_gemm", None) or not self._peer_gather:
            return "separate"
        return (f"ft_ag_gemm (all-gather fused into the first GEMM of {len(self._first_gemm)} of "
                f"{self.num_units} units, {self.first_gemm_calls} calls so far)")

    def shard_range(self):
        return self.rank * self.shard_numel, (self.rank + 1) * self.shard_numel

    def unit_group(self, unit: int) -> ContiguousParaGroup:
        return self._unit_groups[unit]

    def unit_layers(self, unit: int):
        return self._unit_layers[unit]

    def _data_id(self, unit: int):
        return FlexTrainDataID(FlexTrainDataType.PARA, unit)

    # --------------------------------------------------------- init / load
    @torch.no_grad()
    def init_unit_parameters(self, num_layers: int, unit_index: int,
                             layers: Sequence[torch.nn.Module],
                             params: Sequence[torch.nn.Parameter], grouping: Sequence[int]):
        """Flatten one unit, keep this rank's shard in its tiers and take the
        storage away from the module."""
        group = ContiguousParaGroup(params, grouping)
        if not self._initialized:
            self._init_coordinator(num_layers, group.numel)
        if group.numel > self.unit_numel:
            raise ValueError("every unit must hold at most as many parameters as the first one")
        self._unit_groups[unit_index] = group
        self._unit_layers[unit_index] = list(layers)
        self._note_first_gemm(unit_index, layers, group)
        buf = self._buffers[0]
        for p, off, n in zip(group.paras, group.offsets, group.numels):
            buf[off:off + n].copy_(p.data.reshape(-1))
        if group.numel < self.aligned_unit_numel:
            buf[group.numel:].zero_()
        lo, hi = self.shard_range()
        self.write_shard(unit_index, buf[lo:hi])
        self.streams.synchronize()
        for p in group.paras:
            p.data = torch.empty(0, dtype=self.device_dtype, device=self.device)

    def finish_init(self):
        if self._initialized and len(self._unit_groups) != self.num_units:
            raise RuntimeError(f"expected {self.num_units} units, got {len(self._unit_groups)}")

    @torch.no_grad()
    def write_shard(self, unit: int, shard: torch.Tensor):
        """Store a full local shard (device tensor, device dtype) into the tiers."""
        g, c, n = self.tier_numels
        if g:
            if unit not in self._gpu_base:
                self._gpu_base[unit] = allocate_memory(g, self.device_dtype, self.device)
            self._gpu_base[unit].copy_(shard[:g])
        if c:
            if unit not in self._cpu_base:
                self._cpu_base[unit] = allocate_memory(c, self.device_dtype, "cpu", True)
            self._cpu_base[unit].copy_(shard[g:g + c])
        if n:
            land = self._nvme_landing[0]
            land.copy_(shard[g + c:])
            self.streams.synchronize()
            get_nvme_swapper().swap_out(self._data_id(unit), land)

    @torch.no_grad()
    def read_shard(self, unit: int, out: torch.Tensor):
        """Assemble the local shard of ``unit`` into ``out`` (any dtype/device)."""
        g, c, n = self.tier_numels
        self.wait_host_updates(unit)
        if g:
            self._gpu_base_ready.get(unit, DONE).wait()
            out[:g].copy_(self._gpu_base[unit])
        if c:
            out[g:g + c].copy_(self._cpu_base[unit])
        if n:
            land = self._nvme_landing[0]
            get_nvme_swapper().swap_in(self._data_id(unit), land)
            out[g + c:].copy_(land)
            self.streams.synchronize()
        return out

    # -------------------------------------------------- tier views (updates)
    def gpu_base(self, unit: int) -> Optional[torch.Tensor]:
        return self._gpu_base.get(unit)

    def cpu_base(self, unit: int) -> Optional[torch.Tensor]:
        return self._cpu_base.get(unit)

    def note_gpu_base_write(self, unit: int, event: Event):
        self._gpu_base_ready[unit] = event

    def add_host_update(self, unit: int, handle: Waitable):
        self._host_ready.setdefault(unit, []).append(handle)

    def wait_host_updates(self, unit: int):
        for h in self._host_ready.pop(unit, []):
            h.wait()

    def write_nvme_piece(self, unit: int, pinned_piece: torch.Tensor, async_op=False):
        """Replace the NVMe-resident piece of ``unit`` (whole piece)."""
        return get_nvme_swapper().swap_out(self._data_id(unit), pinned_piece, async_op)

    # ------------------------------------------------------------- gather
    def submit_nvme_load(self, unit: int):
        """Start reading the NVMe piece of ``unit`` into a landing buffer."""
        if not self.tier_numels[2] or unit in self._nvme_loads or not 0 <= unit < self.num_units:
            return
        idx = self._nvme_next
        self._nvme_next = (idx + 1) % len(self._nvme_landing)
        # the landing buffer may still feed the H2D copy of an earlier unit, or hold a
        # piece that was read ahead and never consumed
        self._landing_busy[idx].synchronize()
        for other, (i, handle) in list(self._nvme_loads.items()):
            if i == idx:
                handle.wait()
                del self._nvme_loads[other]
        self.wait_host_updates(unit)
        handle = get_nvme_swapper().swap_in(self._data_id(unit), self._nvme_landing[idx], async_op=True)
        self._nvme_loads[unit] = (idx, handle)

    @torch.no_grad()
    def submit_gather(self, unit: int):
        """Queue the assembly + all-gather of ``unit`` into a free ring buffer."""
        if unit in self._inflight or unit in self._held or not 0 <= unit < self.num_units:
            return
        if self._direct:
            # nothing to copy; what has to be awaited (host updates that still write into the
            # base copy) is awaited when the unit is taken, not here, so that a prefetch of the
            # next unit never blocks the launch of the current one
            self._inflight[unit] = (-1, None)
            return
        if unit in self._cached:
            self._inflight[unit] = self._cached.pop(unit)
            return
        if not self._free:
            if not self._cached:
                raise RuntimeError("no free unit buffer: release a unit before gathering another "
                                   "or raise engine.num_unit_buffers")
            oldest = next(iter(self._cached))
            self._free.append(self._cached.pop(oldest))
        idx, free_ev = self._free.popleft()
        buf = self._buffers[idx]
        g, c, n = self.tier_numels
        lo, hi = self.shard_range()
        self.wait_host_updates(unit)
        if n:
            self.submit_nvme_load(unit)
            land_idx, handle = self._nvme_loads.pop(unit)
            handle.wait()
        st = self.streams
        with st.h2d.use():
            st.h2d.wait(free_ev)
            shard = buf[lo:hi]
            if g:
                st.h2d.wait(self._gpu_base_ready.get(unit, DONE))
                tier_copy(shard[:g], self._gpu_base[unit])
            if c:
                tier_copy(shard[g:g + c], self._cpu_base[unit])
            if n:
                tier_copy(shard[g + c:], self._nvme_landing[land_idx])
                self._landing_busy[land_idx] = st.h2d.record()
            if self.world > 1:
                self._all_gather(buf, shard, idx, unit)
            ready = st.h2d.record()
        self._inflight[unit] = (idx, ready)

    def _all_gather(self, buf: torch.Tensor, shard: torch.Tensor, idx: int = -1, unit: int = -1):
        if self.world > 1:
            from .. import TRAFFIC
            TRAFFIC.add("gather", (self.world - 1) * self.shard_numel * self.itemsize)
        self._first_gemm_pending.pop(idx, None)
        if self._peer_gather and idx >= 0:
            from ...parallel import fused
            page = self._flag_page
            ptrs, flags = self._symm[idx].ptr_array(), page.ptr_array()
            shard_bytes = self.shard_numel * self.itemsize
            blocks = self._cfg.engine.fused_blocks
            first = self._first_gemm.get(unit) if self._first_gemm_on else None
            if first is None:
                fused.peer_gather(self.world, self.rank, ptrs, flags, page.next_seq("gather"), shard_bytes,
                                  num_copiers=blocks)
                return
            # everything but the first matrix now; that one arrives inside the product that uses it
            _p, w_lo, rows, cols = first
            w_hi = w_lo + rows * cols * self.itemsize
            total = shard_bytes * self.world
            for lo, hi in ((0, w_lo), (w_hi, total)):
                if hi > lo:
                    fused.peer_gather_range(self.world, self.rank, ptrs, flags, page.next_seq("gather"),
                                            shard_bytes, lo, hi, num_copiers=blocks)
            self._first_gemm_pending[idx] = unit
        else:
            dist.all_gather(buf, shard)

    def _run_first_gemm(self, unit: int, idx: int, x2: torch.Tensor, out: torch.Tensor):
        """``out = x2 @ W.T`` for the unit's first matrix, gathering it into ring buffer ``idx``
        on the way (compute stream; every rank calls it at the same point of its step)."""
        from ...parallel import fused
        _p, w_lo, rows, cols = self._first_gemm[unit]
        page = self._flag_page
        fused.ag_gemm(self.world, self.rank, self._symm[idx].ptr_array(), page.ptr_array(),
                      page.next_seq("ag"), x2, rows, out=out, w_off_bytes=w_lo,
                      shard_bytes=self.shard_numel * self.itemsize)
        self.first_gemm_calls += 1
        from .. import TRAFFIC
        TRAFFIC.add("gather_in_gemm", rows * cols * self.itemsize * (self.world - 1) // self.world)

    def acquire(self, unit: int):
        """Block the compute stream until ``unit`` is gathered; link its parameters."""
        if unit in self._held:
            return
        if unit not in self._inflight:
            self.submit_gather(unit)
        idx, ready = self._inflight.pop(unit)
        if idx < 0:
            # computing straight from the base copy: the host share of the last update must have
            # landed in it (the worker records the event of its copy before it reports done)
            self.wait_host_updates(unit)
            ready = self._gpu_base_ready.get(unit, DONE)
        self.streams.compute.wait(ready)
        self._unit_groups[unit].link_para_to(self._gpu_base[unit] if idx < 0 else self._buffers[idx])
        self._held[unit] = idx
        self._held_version[unit] = self._version.get(unit, 0)
        if idx >= 0 and self._first_gemm_pending.get(idx) == unit:
            self._first_gemm[unit][0]._ft_gather = _PendingFirstGemm(self, unit, idx)

    def release(self, unit: int, keep: bool = False):
        """Unlink ``unit`` and give its buffer back behind a compute-stream
        event.  With ``keep`` the gathered copy stays valid until the buffer is
        needed or ``invalidate(unit)`` is called, so a snake turn that comes
        back to the same unit does not gather it twice."""
        idx = self._held.pop(unit, None)
        if idx is None:
            return
        for p in self._unit_groups[unit].paras:
            p.data = torch.empty(0, dtype=self.device_dtype, device=self.device)
        if idx < 0:
            return
        if self._first_gemm_pending.get(idx) == unit:
            # the unit was let go before any product used its first matrix (a drained prefetch):
            # the buffer is incomplete and must not be kept as a gathered copy
            self._first_gemm_pending.pop(idx, None)
            self._first_gemm[unit][0]._ft_gather = None
            keep = False
        ev = self.streams.compute.record()
        fresh = self._held_version.pop(unit, 0) == self._version.get(unit, 0)
        if keep and fresh and self.num_buffers > 2:
            self._cached[unit] = (idx, ev)
        else:
            self._free.append((idx, ev))

    def invalidate(self, unit: int):
        """The stored shard of ``unit`` is about to change: drop gathered copies."""
        self._version[unit] = self._version.get(unit, 0) + 1
        if unit in self._cached:
            self._free.append(self._cached.pop(unit))

    def held_buffer(self, unit: int) -> torch.Tensor:
        idx = self._held[unit]
        return self._gpu_base[unit] if idx < 0 else self._buffers[idx]

    def detach_all_parameters(self):
        for u in list(self._held):
            self.release(u)

    def drain(self):
        """Drop every in-flight gather (end of step / before re-planning)."""
        for unit in list(self._inflight):
            idx, ready = self._inflight.pop(unit)
            if idx >= 0:
                self._free.append((idx, ready))
        for unit in list(self._cached):
            self._free.append(self._cached.pop(unit))
        self.detach_all_parameters()

    def close(self):
        if self._initialized and self._symm:
            self.streams.synchronize()
            self._buffers = []
            for sb in self._symm:
                sb.close()
            self._symm = []

    # ----------------------------------------------------------- accounting
    def hbm_bytes(self) -> int:
        g = self.tier_numels[0]
        return (self.num_buffers * self.aligned_unit_numel + g * self.num_units) * self.itemsize


_PARA: Optional[FlexTrainParaCoordinator] = None


def get_para_coordinator() -> FlexTrainParaCoordinator:
    global _PARA
    if _PARA is None:
        _PARA = FlexTrainParaCoordinator()
    return _PARA


def reset_para_coordinator():
    global _PARA
    if _PARA is not None and _PARA.is_initialized:
        _PARA.close()
    _PARA = None
