"""Optimizer coordinator: owns the partitioned fp32 master weights and Adam
moments in their tiers, the unit gradient buffers, the gradient reduce-scatter
and the schedule of the device-side and host-side Adam updates.

Parity: flextrain/memory/coordinator/optimizer.py:1-901 (``initialize``
:110-350, alpha split :352-492, ``_submit_transfer_grad`` :534-583, NVMe state
prefetch/offload :585-603,698-731, step planning/execution :605-696, hooks
:733-817, drain :855-888).

Per unit and rank the local shard ``[0, S)`` of fp32 (master, m, v) is cut
``[HBM | DRAM | NVMe]`` by ``split_ratio.optimizer``.  After the last
micro-batch of a unit's backward the opt stream

  1. reduce-scatters the unit gradient (AVG) in place,
  2. optionally raises the unit's non-finite flag,
  3. runs the device Adam kernel on the HBM share (unscale folded in, update
     predicated on the flag, device-dtype parameters written straight into the
     parameter coordinator's HBM base),
  4. copies the rest of the gradient shard to a pinned pool entry and queues
     the host update on a worker thread.

The worker runs the AVX-512 Adam on the DRAM share, streams the NVMe share
through a staging buffer, and writes the updated device-dtype parameters to
where the parameter coordinator keeps them (directly into its pinned base, or
via an H2D copy into its HBM base, or back to the swap file).  Pending host
updates are ordered by unit index ascending - the order in which the next
forward pass needs them - and the size of the pinned gradient pool bounds how
much may be pending: ``alpha`` of the model, the share the reference defers to
the next forward (flextrain/config.py:69-74).  The next gather of a unit waits
for that unit's update only.
"""
from __future__ import annotations

import itertools
import math
import os
import queue
import threading
from concurrent.futures import Future
from typing import Dict, List, Optional

import torch

from ...config import get_flextrain_config
from ...param_group import GroupSegment, create_step_contexts, slice_segments
from ...utils import chaos, distributed as dist
from ...utils.device import DONE, Event, get_streams
from ...utils.logging import rank0_logger
from .. import (tier_copy, FlexTrainDataID, FlexTrainDataType, FutureHandle, allocate_memory,
                get_split_numels)
from ..nvme_swapper import get_nvme_swapper
from .parameter import get_para_coordinator


class _PoolEntry:
    def __init__(self, grad, out, flag):
        self.grad, self.out, self.flag = grad, out, flag


class _HostWorker:
    """One thread that runs host updates, smallest unit index first."""

    def __init__(self):
        self._q: "queue.PriorityQueue" = queue.PriorityQueue()
        self._seq = itertools.count()
        self._thread = threading.Thread(target=self._run, name="ft-host-adam", daemon=True)
        self._device = dist.current_device()
        self._thread.start()

    def submit(self, priority: int, fn) -> Future:
        fut: Future = Future()
        self._q.put((priority, next(self._seq), fn, fut))
        return fut

    def _run(self):
        if self._device.type == "cuda":
            torch.cuda.set_device(self._device)
        while True:
            _prio, _seq, fn, fut = self._q.get()
            if fn is None:
                fut.set_result(None)
                return
            try:
                chaos.perturb("host worker picks up a task")
                fut.set_result(fn())
            except BaseException as exc:      # surfaced by whoever waits on the future
                fut.set_exception(exc)

    def shutdown(self):
        fut: Future = Future()
        self._q.put((1 << 60, next(self._seq), None, fut))
        fut.result()


class FlexTrainOptsCoordinator:
    def __init__(self):
        self._initialized = False

    @property
    def is_initialized(self):
        return self._initialized

    # ----------------------------------------------------------- initialise
    @torch.no_grad()
    def initialize(self, optimizer, loss_scaler):
        cfg = get_flextrain_config()
        para = get_para_coordinator()
        self._cfg, self._para = cfg, para
        self.optimizer = optimizer
        self.cpu_optimizer = optimizer.cpu_optimizer
        self.loss_scaler = loss_scaler
        self.device = dist.current_device()
        self.streams = get_streams()
        self.world, self.rank = dist.get_world_size(), dist.get_rank()
        mp = cfg.mixed_precision
        self.device_dtype = mp.device_dtype
        self.mbpr = cfg.micro_batches_per_rank(self.world)
        self.acc_dtype = mp.gradacc_dtype if (mp.gradacc_dtype != mp.device_dtype and self.mbpr > 1) \
            else None
        self.reduce_dtype = self.acc_dtype or self.device_dtype
        self.check_overflow = mp.device_dtype == torch.float16 or loss_scaler.dynamic
        # Deferred mode: every update waits for the end of backward, when the global gradient
        # norm and one overflow verdict for the whole step exist (strict overflow handling,
        # gradient clipping).  The reduced shards are held until then; nothing overlaps backward.
        self.clip = float(cfg.engine.gradient_clipping)
        self.deferred = bool(cfg.engine.strict_overflow) or self.clip > 0
        self._held: Dict[int, torch.Tensor] = {}
        self._held_scale: Dict[int, float] = {}
        self.last_grad_norm: Optional[float] = None
        self.num_units = para.num_units
        S = para.shard_numel
        self.S = S
        self.K = 1 + optimizer.optimizer_state_per_element
        og, oc, on = get_split_numels(S, cfg.split_ratio.optimizer, 4)
        g, c, n = para.tier_numels
        if n and og > g + c:
            raise ValueError("the HBM share of the optimizer state may not cover NVMe-resident "
                             "parameters: lower split_ratio.optimizer[0] or parameter's NVMe share")
        self.opt_tiers, self.para_tiers = (og, oc, on), (g, c, n)
        self.host_numel = S - og

        # gradient buffers (autograd target) and optional wide accumulators; the buffer the
        # reduction reads is peer-mapped when the fused reduce-scatter kernel is in use
        unit = para.aligned_unit_numel
        self._fused = self._want_fused(cfg, S, og, min(g, og))
        self._symm = []
        self._flag_page = None

        def grad_buffer(dtype, symmetric):
            if not symmetric:
                return allocate_memory(unit, dtype, self.device, zero=True)
            from ...parallel.symm_mem import SymmetricBuffer
            itemsize = torch.empty((), dtype=dtype).element_size()
            sb = SymmetricBuffer(unit * itemsize)
            self._symm.append(sb)
            return sb.tensor(dtype)

        self._grad_bufs = [grad_buffer(self.device_dtype, self._fused and self.acc_dtype is None)
                           for _ in range(2)]
        self._acc_bufs = [grad_buffer(self.acc_dtype, self._fused)
                          for _ in range(2)] if self.acc_dtype is not None else None
        if self._fused:
            from ...parallel.symm_mem import get_flag_page
            self._flag_page = get_flag_page()
            # _symm holds the reduce-source buffers in order [buf0, buf1]
            self._reduce_symm = self._symm[-2:]
        self._buf_free: List[Event] = [DONE, DONE]
        self._buf_next = 0
        self._linked: Dict[int, int] = {}

        # state tiers
        self._gpu_opts: Dict[int, List[torch.Tensor]] = {}
        self._cpu_opts: Dict[int, List[torch.Tensor]] = {}
        # Two sets of staging buffers for the NVMe share of the state: the host update of one unit
        # leaves its write-back in flight and the next unit's update works in the other set, so
        # the disk's write time (its slowest direction) overlaps the next update instead of
        # standing between two of them.  _nvme_stage (set 0) serves start-up and state access.
        self._nvme_stage_sets = [[allocate_memory(on, torch.float32, "cpu", True) for _ in range(self.K)]
                                 for _ in range(2)] if on else None
        self._nvme_stage = self._nvme_stage_sets[0] if on else None
        self._nvme_writes = [None, None]             # (unit, handle) of the write in flight per set
        self._nvme_turn = 0
        self._nvme_para_stage = allocate_memory(n, self.device_dtype, "cpu", True) if n else None
        for stage in [t for ss in (self._nvme_stage_sets or []) for t in ss] + \
                ([self._nvme_para_stage] if n else []):
            get_nvme_swapper().register_staging(stage)
        lo, hi = para.shard_range()
        self._segments: List[List[GroupSegment]] = [
            slice_segments(optimizer.unit_group_segments[u], lo, hi) for u in range(self.num_units)]
        tmp = allocate_memory(S, torch.float32, self.device)
        for u in range(self.num_units):
            para.read_shard(u, tmp)
            if og:
                self._gpu_opts[u] = [allocate_memory(og, torch.float32, self.device, zero=(k > 0))
                                     for k in range(self.K)]
                self._gpu_opts[u][0].copy_(tmp[:og])
            if oc:
                self._cpu_opts[u] = [allocate_memory(oc, torch.float32, "cpu", pinned=False,
                                                     zero=(k > 0)) for k in range(self.K)]
                self._cpu_opts[u][0].copy_(tmp[og:og + oc])
            if on:
                self._nvme_stage[0].copy_(tmp[og + oc:])
                for k in range(1, self.K):
                    self._nvme_stage[k].zero_()
                self.streams.synchronize()
                self._write_nvme_states(u)
        del tmp

        # cross-tier staging: device Adam output that belongs in pinned DRAM
        self._dev_out_stage = None
        if og > g:
            self._dev_out_stage = [allocate_memory(og - g, self.device_dtype, self.device)
                                   for _ in range(2)]
        # host side: pinned gradient pool + worker
        self._pool: "queue.Queue[_PoolEntry]" = queue.Queue()
        self._worker = None
        if self.host_numel:
            depth = max(2, int(math.ceil(cfg.split_ratio.alpha * self.num_units)) + 1)
            out_numel = max(0, min(g, S) - og)        # host-updated parameters that live in HBM
            for _ in range(depth):
                self._pool.put(_PoolEntry(
                    allocate_memory(self.host_numel, self.reduce_dtype, "cpu", True),
                    allocate_memory(out_numel, self.device_dtype, "cpu", True) if out_numel else None,
                    allocate_memory(1, torch.int32, "cpu", True, zero=True)))
            self._pool_depth = depth
            self._worker = _HostWorker()
            threads = cfg.engine.cpu_adam_threads or max(1, (os.cpu_count() or 1) // self.world - 1)
            self.cpu_optimizer.threads = threads
        self._flags = torch.zeros(self.num_units + 1, dtype=torch.int32, device=self.device)
        self._sumsq = torch.zeros(self.num_units, dtype=torch.float32, device=self.device)
        self._host_overflow = False
        self.fused_timeouts = 0            # host updates dropped because their reduction timed out
        self._pending: List[Future] = []
        self.bytes_d2h = 0
        self._initialized = True
        rank0_logger.info(
            f"optimizer geometry: shard={S} state tiers(HBM,DRAM,NVMe)={self.opt_tiers} "
            f"reduce dtype={self.reduce_dtype} overflow check={self.check_overflow} "
            f"host pool depth={getattr(self, '_pool_depth', 0)}")

    def _want_fused(self, cfg, S, og, a_hi) -> bool:
        want = cfg.engine.fused_collectives
        if want is False or self.device.type != "cuda":
            return False
        from ...parallel.symm_mem import peer_access_available
        ok = S % 8 == 0 and og % 8 == 0 and a_hi % 8 == 0 and self.world <= 8 and \
            peer_access_available()
        if want is True and not ok:
            raise RuntimeError("engine.fused_collectives=true needs peer access between all ranks, "
                               "at most 8 ranks and shard / tier sizes that are multiples of 8")
        return bool(ok)

    def _opts_id(self, unit):
        return FlexTrainDataID(FlexTrainDataType.OPTS, unit)

    def _write_nvme_states(self, unit, stage=None, async_op=False):
        from ..nvme_swapper import NVMeGroup
        on = self.opt_tiers[2]
        return NVMeGroup([on] * self.K).group_offload(self._opts_id(unit), stage or self._nvme_stage,
                                                      async_op=async_op)

    def _read_nvme_states(self, unit, stage=None):
        from ..nvme_swapper import NVMeGroup
        on = self.opt_tiers[2]
        self._nvme_settle(unit=unit)                 # never read a file whose write is still in flight
        NVMeGroup([on] * self.K).group_reload(self._opts_id(unit), stage or self._nvme_stage)

    def _nvme_settle(self, which=None, unit=None):
        """Wait for write-backs in flight: of staging set ``which``, of ``unit``'s file, or (no
        argument) all of them.  Called by the thread that owns the sets at that moment: the host
        worker during updates, the main thread once ``wait_all`` has seen the worker idle."""
        for i in range(2):
            pend = self._nvme_writes[i]
            if pend is None or (which is not None and i != which) or (unit is not None and pend[0] != unit):
                continue
            self._nvme_writes[i] = None
            pend[1].wait()

    # ------------------------------------------------------- gradient hooks
    def pre_unit_backward(self, unit: int):
        """Bind the unit's ``.grad`` views to a zeroed gradient buffer."""
        i = self._buf_next
        self._buf_next = (i + 1) % 2
        self.streams.compute.wait(self._buf_free[i])
        self._grad_bufs[i].zero_()
        if self._acc_bufs is not None:
            self._acc_bufs[i].zero_()
        self._para.unit_group(unit).link_grad_to(self._grad_bufs[i])
        self._linked[unit] = i

    @torch.no_grad()
    def post_micro_batch_backward(self, unit: int):
        """Fold the micro-batch gradient into the wide accumulator."""
        if self._acc_bufs is None:
            return
        i = self._linked[unit]
        from ...ops.elementwise import accumulate_and_zero
        accumulate_and_zero(self._acc_bufs[i], self._grad_bufs[i])

    @torch.no_grad()
    def post_unit_backward(self, unit: int):
        """All micro-batches of ``unit`` are back-propagated: reduce, update."""
        i = self._linked.pop(unit)
        self._para.unit_group(unit).detach_grad()
        src = self._acc_bufs[i] if self._acc_bufs is not None else self._grad_bufs[i]
        st = self.streams
        produced = st.compute.record()
        og, oc, on = self.opt_tiers
        g, c, n = self.para_tiers
        lo, hi = self._para.shard_range()
        step = max(int(self.optimizer.param_groups[0]["step"]), 1)
        grad_scale = 1.0 / float(self.loss_scaler.loss_scale)
        if self.deferred:
            self._hold_reduced(unit, i, src, produced, step, grad_scale)
            return
        entry = self._pool.get() if self.host_numel else None    # back-pressure on the host side
        self._para.invalidate(unit)
        host_scale = grad_scale
        with st.opt.use():
            st.opt.wait(produced)
            shard = src[lo:hi]
            flag = self._flags[unit:unit + 1] if self.check_overflow else None
            if self.world > 1:
                from .. import TRAFFIC
                TRAFFIC.add("reduce", (self.world - 1) * shard.numel() * shard.element_size())
            if self._fused and self._fused_reduce(unit, i, shard, step, grad_scale, flag, entry):
                host_scale = 1.0                    # the kernel already unscaled what it handed over
            else:
                self._reduce_scatter(shard, src)
                if flag is not None:
                    from ...ops.adam.gpu_adam import nonfinite_flag
                    nonfinite_flag(shard, flag)
                if og:
                    self._device_update(unit, shard, step, grad_scale, flag, i)
                if entry is not None:
                    tier_copy(entry.grad, shard[og:])
            if entry is not None:
                if flag is not None:
                    tier_copy(entry.flag, flag)
                self.bytes_d2h += self.host_numel * entry.grad.element_size()
            done = st.opt.record()
        self._buf_free[i] = done
        if og:
            self._para.note_gpu_base_write(unit, done)
        if entry is not None:
            groups = self._hyper_snapshot()
            fut = self._worker.submit(
                unit, lambda: self._host_update(unit, entry, done, step, host_scale, groups))
            self._para.add_host_update(unit, FutureHandle(fut))
            self._pending.append(fut)

    def _fused_reduce(self, unit, buf_index, shard, step, grad_scale, flag, entry, defer=False) -> bool:
        """One kernel: peer reduce-scatter + unscale (+ Adam on the HBM share and the
        host hand-off when no overflow check has to come first).  Returns False when
        this unit's segments cannot be expressed to the kernel."""
        from ...parallel import fused
        og = self.opt_tiers[0]
        g = self.para_tiers[0]
        segs = slice_segments(self._segments[unit], 0, og, rebase=False)
        a_hi = min(g, og)
        if not fused.segments_aligned(segs, og, a_hi):
            return False
        symm = self._reduce_symm[buf_index]
        page = self._flag_page
        seq = page.next_seq("rs")
        scale = grad_scale / self.world
        two_phase = flag is not None
        if flag is not None:
            flag.zero_()
        # where a rank that gave up waiting for its peers says so: the unit's skip flag when the
        # update waits for it anyway, else the pinned word the host worker reads before it
        # touches any state (nothing was reduced or handed over in that case)
        status = flag if two_phase else (entry.flag if entry is not None else None)
        if entry is not None and not two_phase:
            entry.flag.zero_()
        opts = self._gpu_opts.get(unit)
        stage = self._dev_out_stage[buf_index] if self._dev_out_stage is not None else None
        fused.rs_adam(
            self.world, self.rank, symm.ptr_array(), page.ptr_array(), self.reduce_dtype, self.S, scale,
            seq, reduced_out=shard if two_phase else None, og=og, do_adam=(not two_phase) and og > 0,
            master=opts[0] if opts else None, m=opts[1] if opts else None, v=opts[2] if opts else None,
            param_a=self._para.gpu_base(unit), a_hi=a_hi, param_b=stage, param_dtype=self.device_dtype,
            host_grad=None if (two_phase or entry is None) else entry.grad, finite_flag=flag,
            segments=fused.make_segments(segs, self.optimizer.param_groups, self.cpu_optimizer, step),
            nseg=len(segs), max_blocks=self._cfg.engine.fused_blocks, status=status)
        if defer:
            return True                             # the caller keeps the reduced shard
        if two_phase:
            if og:
                self._device_update(unit, shard, step, 1.0, flag, buf_index)
            if entry is not None:
                tier_copy(entry.grad, shard[og:])
        elif og > g:
            tier_copy(self._para.cpu_base(unit)[: og - g], stage[: og - g])
        return True

    def _reduce_scatter(self, shard: torch.Tensor, full: torch.Tensor):
        dist.reduce_scatter(shard, full, dist.ReduceOp.AVG)

    def _device_update(self, unit, shard, step, grad_scale, flag, buf_index):
        from ...ops.adam.gpu_adam import device_adam_update
        og = self.opt_tiers[0]
        g = self.para_tiers[0]
        opts = self._gpu_opts[unit]
        gpu_base = self._para.gpu_base(unit)
        stage = self._dev_out_stage[buf_index] if self._dev_out_stage is not None else None
        cuts = sorted({0, min(g, og), og})
        for a, b in zip(cuts[:-1], cuts[1:]):
            if b <= a:
                continue
            for seg in slice_segments(self._segments[unit], a, b, rebase=False):
                sl = slice(seg.start, seg.end)
                if seg.end <= g:
                    out = gpu_base[sl]
                else:
                    out = stage[seg.start - g:seg.end - g]
                device_adam_update(self.optimizer.param_groups[seg.group], step, self.cpu_optimizer,
                                   opts[0][sl], shard[sl], [o[sl] for o in opts[1:]], out,
                                   grad_scale=grad_scale, skip_flag=flag)
        if og > g:
            # parameters updated on the device but resident in pinned DRAM
            tier_copy(self._para.cpu_base(unit)[: og - g], stage[: og - g])

    # ---------------------------------------------------------- host update
    def _hyper_snapshot(self):
        """Hyper-parameters of every param group as they are now.  A host update runs later,
        possibly during the next step's forward: it must use the rates of the step whose
        gradients it applies, not whatever a scheduler has written since."""
        return [{k: v for k, v in g.items() if k != "params"} for g in self.optimizer.param_groups]

    def _host_update(self, unit, entry: _PoolEntry, grads_ready: Event, step, grad_scale, groups=None):
        try:
            grads_ready.synchronize()
            chaos.perturb("host update has its gradients")
            word = int(entry.flag.item())
            if word != 0:
                # non-finite gradient (1) or a fused reduction that gave up at its start barrier
                # (101): the pool entry holds no gradient of this unit, no state may change
                if word == 101:
                    self.fused_timeouts += 1
                else:
                    self._host_overflow = True
                return
            og, oc, on = self.opt_tiers
            g, c, n = self.para_tiers
            para = self._para
            if groups is None:
                groups = self.optimizer.param_groups
            segs = self._segments[unit]
            # device-dtype destinations, in shard coordinates
            out_hbm_hi = max(og, min(g, self.S))     # [og, out_hbm_hi) -> entry.out -> gpu_base
            cpu_base = para.cpu_base(unit)

            def out_view(a, b):
                if b <= out_hbm_hi:
                    return entry.out[a - og:b - og]
                if a >= g + c:
                    return self._nvme_para_stage[a - g - c:b - g - c]
                return cpu_base[a - g:b - g]

            def run(region_lo, region_hi, master, states, base):
                cuts = sorted({region_lo, region_hi,
                               *[x for x in (out_hbm_hi, g, g + c) if region_lo < x < region_hi]})
                for a, b in zip(cuts[:-1], cuts[1:]):
                    for seg in slice_segments(segs, a, b, rebase=False):
                        sl = slice(seg.start - base, seg.end - base)
                        ctxs = create_step_contexts(
                            groups, [GroupSegment(seg.group, 0, seg.numel)], master[sl],
                            entry.grad[seg.start - og:seg.end - og], [s[sl] for s in states],
                            out_view(seg.start, seg.end))
                        self.cpu_optimizer.step(ctxs, step=step, grad_scale=grad_scale)

            if oc:
                opts = self._cpu_opts[unit]
                run(og, og + oc, opts[0], opts[1:], og)
            if on:
                i = self._nvme_turn
                self._nvme_turn ^= 1
                stage = self._nvme_stage_sets[i]
                self._nvme_settle(which=i)           # the write that last used this set
                self._read_nvme_states(unit, stage)
                run(og + oc, self.S, stage[0], stage[1:], og + oc)
                self._nvme_writes[i] = (unit, self._write_nvme_states(unit, stage, async_op=True))
            if n:
                para.write_nvme_piece(unit, self._nvme_para_stage)
            if out_hbm_hi > og:
                st = self.streams
                with st.h2d.use():
                    para.gpu_base(unit)[og:out_hbm_hi].copy_(entry.out[: out_hbm_hi - og],
                                                             non_blocking=True)
                    ev = st.h2d.record()
                chaos.perturb("host update copied back, not yet announced")
                para.note_gpu_base_write(unit, ev)
                ev.synchronize()
        finally:
            self._pool.put(entry)

    # ------------------------------------------------------------ deferred mode
    def _hold_reduced(self, unit, i, src, produced, step, grad_scale):
        """Deferred mode: reduce-scatter ``unit``'s gradients, keep the reduced
        shard and its squared norm; no update yet."""
        st = self.streams
        lo, hi = self._para.shard_range()
        with st.opt.use():
            st.opt.wait(produced)
            shard = src[lo:hi]
            flag = self._flags[unit:unit + 1]
            if self._fused and self._fused_reduce(unit, i, shard, step, grad_scale, flag, None, defer=True):
                held_scale = 1.0                     # the kernel unscaled and averaged already
            else:
                self._reduce_scatter(shard, src)
                held_scale = grad_scale
            hold = self._held.get(unit)
            if hold is None:
                hold = allocate_memory(self.S, shard.dtype, self.device)
                self._held[unit] = hold
            hold.copy_(shard)
            self._sumsq[unit] = torch.linalg.vector_norm(hold, dtype=torch.float32) ** 2 * (held_scale ** 2)
            done = st.opt.record()
        self._buf_free[i] = done
        self._held_scale[unit] = held_scale

    @torch.no_grad()
    def resolve_deferred(self, extra_sumsq=0.0):
        """End of a deferred step: global gradient norm over every unit shard of
        every rank plus ``extra_sumsq`` (the replicated parameters' share), one
        overflow verdict, the clip coefficient, then the held updates in
        ascending unit order (the order the next forward needs them).
        Returns ``(overflow, clip_coefficient)``."""
        st = self.streams
        with st.opt.use():
            total = self._sumsq.sum()
            done = st.opt.record()
        done.synchronize()
        total = dist.all_reduce_scalar(float(total), dist.ReduceOp.SUM) if self.world > 1 else float(total)
        total += float(extra_sumsq)
        overflow = not math.isfinite(total)
        coef = 1.0
        if not overflow:
            norm = math.sqrt(max(total, 0.0))
            self.last_grad_norm = norm
            if self.clip > 0:
                coef = min(1.0, self.clip / (norm + 1e-6))
            step = max(int(self.optimizer.param_groups[0]["step"]), 1)
            for unit in sorted(self._held_scale):
                self._apply_held(unit, step, coef)
        self._held_scale.clear()
        return overflow, coef

    def _apply_held(self, unit, step, coef):
        st = self.streams
        og = self.opt_tiers[0]
        hold = self._held[unit]
        scale = self._held_scale[unit] * coef
        entry = self._pool.get() if self.host_numel else None
        self._para.invalidate(unit)
        with st.opt.use():
            if og:
                self._device_update(unit, hold, step, scale, None, unit % 2)
            if entry is not None:
                tier_copy(entry.grad, hold[og:])
                entry.flag.zero_()
            done = st.opt.record()
        if og:
            self._para.note_gpu_base_write(unit, done)
        if entry is not None:
            groups = self._hyper_snapshot()
            fut = self._worker.submit(
                unit, lambda u=unit, e=entry, d=done, sc=scale, g=groups: self._host_update(u, e, d, step, sc, g))
            self._para.add_host_update(unit, FutureHandle(fut))
            self._pending.append(fut)

    # -------------------------------------------------------------- end of step
    def finish_step(self) -> bool:
        """Called once per iteration after backward.  Returns True if any unit
        met a non-finite gradient (its update was skipped)."""
        overflow = False
        if self.check_overflow:
            # the flags are raised on the optimizer stream (reduce kernel / finite check of the
            # last units are still running when backward has been launched): read them there
            with self.streams.opt.use():
                any_flag = self._flags.any()
                read = self.streams.opt.record()
            read.synchronize()
            overflow = bool(any_flag.item())
        return overflow

    def collect_host_overflow(self) -> bool:
        """Wait for every queued host update and report host-side overflow."""
        self.wait_all()
        flag, self._host_overflow = self._host_overflow, False
        return flag

    def wait_all(self):
        pend, self._pending = self._pending, []
        for f in pend:
            f.result()
        if getattr(self, "_nvme_stage_sets", None):
            self._nvme_settle()

    def prune_pending(self):
        done = [f for f in self._pending if f.done()]
        for f in done:
            f.result()
        self._pending = [f for f in self._pending if not f.done()]

    def shutdown(self):
        if self._worker is not None:
            self.wait_all()
            self._worker.shutdown()
            self._worker = None
        if getattr(self, "_symm", None):
            self.streams.synchronize()
            self._grad_bufs, self._acc_bufs = [], None
            for sb in self._symm:
                sb.close()
            self._symm = []

    # ---------------------------------------------------------- state access
    @torch.no_grad()
    def read_states(self, unit: int) -> List[torch.Tensor]:
        """fp32 (master, m, v) of the local shard as CPU tensors (save / tests)."""
        self.wait_all()
        self.streams.synchronize()
        og, oc, on = self.opt_tiers
        out = [torch.empty(self.S, dtype=torch.float32) for _ in range(self.K)]
        for k in range(self.K):
            if og:
                out[k][:og].copy_(self._gpu_opts[unit][k])
            if oc:
                out[k][og:og + oc].copy_(self._cpu_opts[unit][k])
        if on:
            self._read_nvme_states(unit)
            for k in range(self.K):
                out[k][og + oc:].copy_(self._nvme_stage[k])
        return out

    @torch.no_grad()
    def write_states(self, unit: int, states: List[torch.Tensor]):
        self.wait_all()
        og, oc, on = self.opt_tiers
        for k in range(self.K):
            if og:
                self._gpu_opts[unit][k].copy_(states[k][:og])
            if oc:
                self._cpu_opts[unit][k].copy_(states[k][og:og + oc])
            if on:
                self._nvme_stage[k].copy_(states[k][og + oc:])
        if on:
            self._write_nvme_states(unit)
        shard = states[0].to(self.device).to(self.device_dtype)
        self._para.invalidate(unit)
        self._para.write_shard(unit, shard)
        self.streams.synchronize()


_OPTS: Optional[FlexTrainOptsCoordinator] = None


def get_opts_coordinator() -> FlexTrainOptsCoordinator:
    global _OPTS
    if _OPTS is None:
        _OPTS = FlexTrainOptsCoordinator()
    return _OPTS


def reset_opts_coordinator():
    global _OPTS
    if _OPTS is not None and _OPTS.is_initialized:
        _OPTS.shutdown()
    _OPTS = None
