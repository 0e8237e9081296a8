"""Optimizer front-end: maps param groups onto the partitioned unit buffers and
owns the parameters that live outside the layer stack.

Parity: flextrain/optimizer.py:1-272 - ``FlexTrainCPUOptimizer`` ABC :24-95
(``_init_optimizer_states``, ``_step``, ``step(step_contexts)``,
``profile_step``), ``FlexTrainOptimizer`` :98-272 (param -> group map, per-unit
``GroupSegment`` lists, non-layerwise parameters in one contiguous device
buffer with fp32 master and states, ``step`` = all-reduce AVG -> Adam -> copy
back, ``update_states`` increments ``group["step"]``).

Differences: ``param_groups`` may also be a plain iterable of tensors; the
non-layerwise parameters are stepped on the device when their state fits there
(the reference always round-trips them through the host), with gradient
unscaling and the overflow flag folded into the same kernel.
"""
from __future__ import annotations

import time
from abc import ABC, abstractmethod
from typing import Dict, List, Optional, Sequence

import torch

from .param_group import (GroupSegment, StepContext, create_group_segments, create_step_contexts,
                          slice_segments)
from .utils import distributed as dist

STEP_KEY = "step"
PARAMS_KEY = "params"


class FlexTrainCPUOptimizer(ABC):
    """Host optimizer over flat fp32 state.  Sub-classes supply the state
    layout and the fused update of one contiguous range."""

    optimizer_state_per_element = 0

    def __init__(self, param_groups=None):
        self.param_groups_arg = param_groups

    @abstractmethod
    def _init_optimizer_states(self, numel: int, dtype: torch.dtype, pin: bool = False) -> List[torch.Tensor]:
        ...

    @abstractmethod
    def _step(self, ctx: StepContext, step: int, grad_scale: float = 1.0) -> bool:
        ...

    @torch.no_grad()
    def step(self, step_contexts, step: Optional[int] = None, grad_scale: float = 1.0) -> bool:
        """Update every non-empty context.  ``step`` defaults to the group's own
        counter.  Returns True if a non-finite gradient was met."""
        if isinstance(step_contexts, StepContext):
            step_contexts = [step_contexts]
        bad = False
        for ctx in step_contexts:
            if ctx.grad.numel() == 0:
                continue
            s = step if step is not None else int(ctx.group.get(STEP_KEY, 1))
            bad |= bool(self._step(ctx, max(s, 1), grad_scale))
        return bad

    @torch.no_grad()
    def profile_step(self, numel: int, device_dtype: torch.dtype, master_dtype: torch.dtype) -> float:
        """One timed update over ``numel`` synthetic elements; seconds."""
        cache = getattr(self, "_profile", None)
        if cache is None or cache["numel"] != numel:
            cache = dict(numel=numel, group={STEP_KEY: 0, **getattr(self, "defaults", {})},
                         half=torch.empty(numel, dtype=device_dtype),
                         full=torch.randn(numel, dtype=master_dtype),
                         grad=torch.randn(numel, dtype=master_dtype),
                         states=self._init_optimizer_states(numel, master_dtype))
            self._profile = cache
        cache["group"][STEP_KEY] += 1
        ctx = StepContext(cache["group"], cache["full"], cache["grad"], cache["states"], cache["half"])
        t0 = time.perf_counter()
        self._step(ctx, cache["group"][STEP_KEY])
        return time.perf_counter() - t0


def _normalise_param_groups(param_groups, defaults: Dict) -> List[Dict]:
    groups = list(param_groups)
    if not groups:
        raise ValueError("optimizer got an empty parameter list")
    if not isinstance(groups[0], dict):
        groups = [{PARAMS_KEY: groups}]
    out = []
    for g in groups:
        g = dict(g)
        params = g[PARAMS_KEY]
        g[PARAMS_KEY] = [params] if isinstance(params, torch.Tensor) else list(params)
        for k, v in defaults.items():
            g.setdefault(k, v)
        g.setdefault(STEP_KEY, 0)
        out.append(g)
    return out


class FlexTrainOptimizer:
    """Holds the param groups, the per-unit group segments the coordinators
    need, and the optimizer state of the non-layerwise parameters."""

    def __init__(self, param_groups, cpu_optimizer: FlexTrainCPUOptimizer):
        from .config import get_flextrain_config
        from .memory.coordinator.parameter import get_para_coordinator
        self.cpu_optimizer = cpu_optimizer
        self.param_groups: List[Dict] = _normalise_param_groups(param_groups, cpu_optimizer.defaults)
        self.optimizer_state_per_element = cpu_optimizer.optimizer_state_per_element
        cfg = get_flextrain_config()
        para = get_para_coordinator()
        self._cfg = cfg
        self.device = dist.current_device()
        self.device_dtype = cfg.mixed_precision.device_dtype
        self.master_dtype = cfg.mixed_precision.master_dtype

        # ---- parameter -> group index
        group_of: Dict[int, int] = {}
        for gi, g in enumerate(self.param_groups):
            for p in g[PARAMS_KEY]:
                if id(p) in group_of:
                    raise ValueError("a parameter appears in more than one param group")
                group_of[id(p)] = gi

        # ---- layer parameters: segments over each unit's flat buffer
        self.unit_group_segments: List[List[GroupSegment]] = []
        layer_param_ids = set()
        for u in range(para.num_units):
            grp = para.unit_group(u)
            gids = []
            for p in grp.paras:
                layer_param_ids.add(id(p))
                if id(p) not in group_of:
                    raise ValueError("a layer parameter is missing from the optimizer's param groups")
                gids.append(group_of[id(p)])
            segs = create_group_segments(grp.numels, gids)
            # padding up to the aligned unit size follows the last group
            pad = para.aligned_unit_numel - grp.numel
            if pad:
                last = segs[-1].group if segs else 0
                segs = segs + [GroupSegment(last, grp.numel, para.aligned_unit_numel)]
                from .param_group import merge_segments
                segs = merge_segments(segs)
            self.unit_group_segments.append(segs)

        # ---- everything else is replicated on every rank ("non-layerwise")
        self.non_layerwise_params: List[torch.nn.Parameter] = []
        nl_groups: List[int] = []
        for gi, g in enumerate(self.param_groups):
            for p in g[PARAMS_KEY]:
                if id(p) not in layer_param_ids:
                    self.non_layerwise_params.append(p)
                    nl_groups.append(gi)
        self._build_non_layerwise(nl_groups)
        para.detach_all_parameters()

    # ------------------------------------------------------ non-layerwise
    def _build_non_layerwise(self, groups: Sequence[int]):
        params = self.non_layerwise_params
        numels = [p.numel() for p in params]
        total = sum(numels)
        self._nl_numel = total
        self._nl_segments = create_group_segments(numels, groups) if params else []
        if not params:
            return
        from .memory import allocate_memory, move_into_contiguous
        dev = self.device
        where = self._cfg.engine.nonlayer_optimizer_device
        self._nl_on_device = (where == "gpu") or (where == "auto")
        self._nl_fused = self._nl_want_fused()
        world, rank = dist.get_world_size(), dist.get_rank()
        if self._nl_fused:
            # Peer-mapped flat parameter and gradient buffers, padded so that they
            # split into `world` slices of a multiple of 8 elements; the fp32 state
            # exists only for this rank's slice.
            from .parallel.symm_mem import SymmetricBuffer, get_flag_page
            from .param_group import merge_segments
            shard = -(-total // (world * 8)) * 8
            padded = shard * world
            if padded > total:
                last = self._nl_segments[-1].group
                self._nl_segments = merge_segments(
                    list(self._nl_segments) + [GroupSegment(last, total, padded)])
            itemsize = torch.empty((), dtype=self.device_dtype).element_size()
            self._nl_para_symm = SymmetricBuffer(padded * itemsize)
            self._nl_grad_symm = SymmetricBuffer(padded * itemsize)
            self._nl_flag_page = get_flag_page()
            self._nl_para = self._nl_para_symm.tensor(self.device_dtype)
            self._nl_grad = self._nl_grad_symm.tensor(self.device_dtype)
            self._nl_grad.zero_()
            self._nl_shard, self._nl_lo = shard, rank * shard
            state_numel = shard
        else:
            self._nl_para = allocate_memory(total, self.device_dtype, dev)
            self._nl_grad = allocate_memory(total, self.device_dtype, dev, zero=True)
            self._nl_shard, self._nl_lo = total, 0
            state_numel = total
        move_into_contiguous(params, self._nl_para[:total])
        off = 0
        for p, n in zip(params, numels):
            p.grad = self._nl_grad[off:off + n].view(p.shape)
            off += n
        state_dev = dev if self._nl_on_device else torch.device("cpu")
        pinned = not self._nl_on_device
        self._nl_master = allocate_memory(state_numel, self.master_dtype, state_dev, pinned)
        self._nl_master.copy_(self._nl_para[self._nl_lo:self._nl_lo + state_numel])
        self._nl_states = [allocate_memory(state_numel, self.master_dtype, state_dev, pinned, zero=True)
                           for _ in range(self.optimizer_state_per_element)]
        if not self._nl_on_device:
            self._nl_host_grad = allocate_memory(total, torch.float32, "cpu", True)
            self._nl_host_para = allocate_memory(total, self.device_dtype, "cpu", True)
        self._nl_flag = torch.zeros(1, dtype=torch.int32, device=dev)

    def _nl_want_fused(self) -> bool:
        """The fused all-reduce + Adam kernel needs CUDA, the update on the
        device, peer access between all ranks, group boundaries on multiples of
        8 elements and the built-in Adam (it carries its own arithmetic)."""
        want = self._cfg.engine.fused_collectives
        if want is False or self.device.type != "cuda" or not self._nl_on_device:
            return False
        if self._cfg.engine.strict_overflow or self._cfg.engine.gradient_clipping > 0:
            return False                            # deferred mode splits reduce and update
        nl = self._cfg.engine.fused_nonlayer
        if nl is False:
            return False
        from .ops.adam import FlexTrainCPUAdam
        from .parallel.fused import segments_aligned
        from .parallel.symm_mem import peer_access_available
        if not isinstance(self.cpu_optimizer, FlexTrainCPUAdam):
            return False
        if self.master_dtype != torch.float32 or self.optimizer_state_per_element != 2:
            return False
        return segments_aligned(self._nl_segments) and dist.get_world_size() <= 8 \
            and peer_access_available()

    def _nl_fused_step(self, grad_scale: float, check_overflow: bool) -> bool:
        """Non-layerwise update as one kernel: every rank reduces its slice of
        all ranks' gradients over NVLink, updates its slice of the fp32 state and
        stores the new parameters into every rank's buffer."""
        from .ops.adam.gpu_adam import device_adam_update
        from .parallel import fused
        from .param_group import slice_segments
        world, rank = dist.get_world_size(), dist.get_rank()
        S, lo = self._nl_shard, self._nl_lo
        segs = slice_segments(self._nl_segments, lo, lo + S, rebase=True)
        page = self._nl_flag_page
        step = max(int(self.param_groups[0][STEP_KEY]), 1)
        arr = fused.make_segments(segs, self.param_groups, self.cpu_optimizer, step)
        for i, seg in enumerate(segs):          # every group carries its own step counter
            arr[i].step = max(int(self.param_groups[seg.group][STEP_KEY]), 1)
        own = self._nl_grad[lo:lo + S]
        if check_overflow:
            self._nl_flag.zero_()
        fused.ar_adam(world, rank, self._nl_grad_symm.ptr_array(), page.ptr_array(), self.device_dtype,
                      S, grad_scale / world, page.next_seq("nl"),
                      reduced_out=own if check_overflow else None, do_adam=not check_overflow,
                      master=self._nl_master, m=self._nl_states[0], v=self._nl_states[1],
                      param_ptrs=self._nl_para_symm.ptr_array(), param_dtype=self.device_dtype,
                      finite_flag=self._nl_flag if check_overflow else None, segments=arr,
                      nseg=len(segs), max_blocks=self._cfg.engine.fused_blocks)
        overflow = False
        if check_overflow:
            overflow = dist.all_reduce_scalar(float(self._nl_flag.item() != 0), dist.ReduceOp.MAX) > 0
            if not overflow:
                for seg in segs:
                    g = self.param_groups[seg.group]
                    sl = slice(seg.start, seg.end)
                    device_adam_update(g, max(int(g[STEP_KEY]), 1), self.cpu_optimizer,
                                       self._nl_master[sl], own[sl], [s[sl] for s in self._nl_states],
                                       self._nl_para[lo:lo + S][sl], grad_scale=1.0)
                itemsize = self._nl_para.element_size()
                fused.peer_gather(world, rank, self._nl_para_symm.ptr_array(), page.ptr_array(),
                                  page.next_seq("nl_gather"), S * itemsize, start_slot=8, done_slot=9)
        self._nl_grad.zero_()
        return overflow

    def fused_nonlayer_in_use(self) -> bool:
        return bool(getattr(self, "_nl_fused", False)) and not getattr(self, "_nl_fused_off", False)

    def disable_fused_nonlayer(self):
        """Stop using the fused all-reduce + Adam kernel (after one of its waits ran out).  The
        fp32 state stays sharded over the ranks; the reduction and the hand-out of the updated
        parameters go through the library collectives from now on."""
        self._nl_fused_off = True

    def _nl_sharded_library_step(self, grad_scale: float, check_overflow: bool) -> bool:
        """The sharded non-layerwise update without the fused kernel: all-reduce (AVG) of the
        gradients, Adam on this rank's slice of the fp32 state, all-gather of the slices."""
        from .ops.adam.gpu_adam import device_adam_update, has_nonfinite
        from .param_group import slice_segments
        S, lo = self._nl_shard, self._nl_lo
        dist.all_reduce(self._nl_grad, dist.ReduceOp.AVG)
        overflow = has_nonfinite(self._nl_grad) if check_overflow else False
        if not overflow:
            own = self._nl_grad[lo:lo + S]
            for seg in slice_segments(self._nl_segments, lo, lo + S, rebase=True):
                g = self.param_groups[seg.group]
                sl = slice(seg.start, seg.end)
                device_adam_update(g, max(int(g[STEP_KEY]), 1), self.cpu_optimizer,
                                   self._nl_master[sl], own[sl], [s[sl] for s in self._nl_states],
                                   self._nl_para[lo:lo + S][sl], grad_scale=grad_scale)
            dist.all_gather(self._nl_para, self._nl_para[lo:lo + S])
        self._nl_grad.zero_()
        return overflow

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0, check_overflow: bool = False) -> bool:
        """Average the replicated gradients over ranks and apply one update to
        the non-layerwise parameters.  Returns True if the step was skipped
        because of a non-finite gradient."""
        if not self.non_layerwise_params:
            return False
        from .ops.adam.gpu_adam import has_nonfinite
        if self._nl_fused:
            if getattr(self, "_nl_fused_off", False):
                return self._nl_sharded_library_step(grad_scale, check_overflow)
            return self._nl_fused_step(grad_scale, check_overflow)
        self.reduce_gradients()
        overflow = has_nonfinite(self._nl_grad) if check_overflow else False
        if overflow:
            self.discard_gradients()
        else:
            self.apply_update(grad_scale)
        return overflow

    @torch.no_grad()
    def reduce_gradients(self):
        """First half of ``step``: average the replicated gradients over ranks."""
        if self.non_layerwise_params:
            dist.all_reduce(self._nl_grad, dist.ReduceOp.AVG)

    @torch.no_grad()
    def gradient_sumsq(self, grad_scale: float = 1.0) -> float:
        """Squared L2 norm of the (reduced, unscaled) non-layerwise gradients."""
        if not self.non_layerwise_params:
            return 0.0
        n = torch.linalg.vector_norm(self._nl_grad, dtype=torch.float32)
        return float(n) ** 2 * float(grad_scale) ** 2

    @torch.no_grad()
    def discard_gradients(self):
        if self.non_layerwise_params:
            self._nl_grad.zero_()

    @torch.no_grad()
    def apply_update(self, grad_scale: float = 1.0):
        """Second half of ``step``: one update from the already reduced gradients
        (``grad_scale`` may carry a clip coefficient), then zero them."""
        if not self.non_layerwise_params:
            return
        from .ops.adam.gpu_adam import device_adam_update
        if self._nl_on_device:
            for seg in self._nl_segments:
                g = self.param_groups[seg.group]
                sl = slice(seg.start, seg.end)
                device_adam_update(g, max(int(g[STEP_KEY]), 1), self.cpu_optimizer,
                                   self._nl_master[sl], self._nl_grad[sl],
                                   [s[sl] for s in self._nl_states], self._nl_para[sl],
                                   grad_scale=grad_scale)
        else:
            self._nl_host_grad.copy_(self._nl_grad)     # synchronous: pageable semantics
            if self.device.type == "cuda":
                torch.cuda.current_stream().synchronize()
            ctxs = create_step_contexts(self.param_groups, self._nl_segments, self._nl_master,
                                        self._nl_host_grad, self._nl_states, self._nl_host_para)
            self.cpu_optimizer.step(ctxs, grad_scale=grad_scale)
            self._nl_para.copy_(self._nl_host_para, non_blocking=True)
        self._nl_grad.zero_()

    @property
    def non_layerwise_numel(self) -> int:
        """Elements of the parameters outside the layer stack (embeddings, final norm, head;
        flextrain/optimizer.py:240-242)."""
        return self._nl_numel

    def close(self):
        """Release the peer-mapped buffers of the fused non-layerwise path (the
        parameters move to ordinary device memory first).  Collective."""
        if not self.non_layerwise_params or not getattr(self, "_nl_fused", False):
            return
        torch.cuda.synchronize()
        keep = self._nl_para[:self._nl_numel].clone()
        off = 0
        for p in self.non_layerwise_params:
            n = p.numel()
            p.data = keep[off:off + n].view(p.shape)
            p.grad = None
            off += n
        self._nl_para, self._nl_grad = keep, None
        self._nl_para_symm.close()
        self._nl_grad_symm.close()
        self._nl_fused = False

    def update_states(self):
        """Advance every group's step counter (once per training iteration)."""
        for g in self.param_groups:
            g[STEP_KEY] += 1

    # -------------------------------------------------- state (save / load)
    def non_layerwise_state(self):
        """fp32 master and moments of the non-layerwise parameters: the whole
        vector when the state is replicated, this rank's slice when the fused
        all-reduce kernel keeps it sharded."""
        if not self.non_layerwise_params:
            return {}
        return {"master": self._nl_master.detach().cpu().clone(),
                "states": [s.detach().cpu().clone() for s in self._nl_states],
                "sharded": bool(self._nl_fused), "total": self._nl_numel, "lo": self._nl_lo}

    def load_non_layerwise_full(self, master: torch.Tensor, states):
        """Install the state from whole vectors (``total`` elements each, any
        rank layout it was saved under): the resharding path of ``engine.load``."""
        if not self.non_layerwise_params:
            return
        total = self._nl_numel
        if master.numel() != total or any(s.numel() != total for s in states):
            raise ValueError("non-layerwise state of the checkpoint does not match this model")
        lo, n = self._nl_lo, self._nl_master.numel()
        hi = min(lo + n, total)

        def piece(full):
            out = torch.zeros(n, dtype=full.dtype)
            if hi > lo:
                out[:hi - lo].copy_(full[lo:hi])
            return out
        self.load_non_layerwise_state({"master": piece(master), "states": [piece(s) for s in states],
                                       "sharded": bool(self._nl_fused)})

    def load_non_layerwise_state(self, state):
        if not state:
            return
        if bool(state.get("sharded", False)) != bool(self._nl_fused):
            raise ValueError("non-layerwise optimizer state was saved with a different "
                             "engine.fused_collectives setting")
        self._nl_master.copy_(state["master"])
        for dst, src in zip(self._nl_states, state["states"]):
            dst.copy_(src)
        lo, n = self._nl_lo, self._nl_master.numel()
        self._nl_para[lo:lo + n].copy_(self._nl_master)
        if self._nl_fused and dist.get_world_size() > 1:
            import torch.distributed as tdist
            tdist.all_gather_into_tensor(self._nl_para, self._nl_para[lo:lo + n].clone())

    def non_layerwise_master_full(self) -> Optional[torch.Tensor]:
        """The fp32 master vector of all non-layerwise parameters on the CPU
        (gathered over ranks when the state is sharded).  Collective."""
        if not self.non_layerwise_params:
            return None
        local = self._nl_master.detach()
        if self._nl_fused and dist.get_world_size() > 1:
            import torch.distributed as tdist
            full = torch.empty(local.numel() * dist.get_world_size(), dtype=local.dtype, device=local.device)
            tdist.all_gather_into_tensor(full, local.contiguous())
            return full[:self._nl_numel].cpu()
        return local[:self._nl_numel].cpu().clone()

    def set_non_layerwise_master(self, full: torch.Tensor, reset_moments: bool = True):
        """Overwrite the master weights (and the 16-bit copies) of the non-layerwise
        parameters from a whole vector; the moments are zeroed or kept."""
        if not self.non_layerwise_params:
            return
        if full.numel() != self._nl_numel:
            raise ValueError("non-layerwise vector does not match this model")
        lo, n = self._nl_lo, self._nl_master.numel()
        hi = min(lo + n, self._nl_numel)
        piece = torch.zeros(n, dtype=torch.float32)
        if hi > lo:
            piece[:hi - lo].copy_(full[lo:hi])
        states = [torch.zeros(n, dtype=torch.float32) if reset_moments else s.detach().cpu()
                  for s in self._nl_states]
        self.load_non_layerwise_state({"master": piece, "states": states, "sharded": bool(self._nl_fused)})

    def hyper_state(self):
        return [{k: v for k, v in g.items() if k != PARAMS_KEY} for g in self.param_groups]

    def load_hyper_state(self, state):
        for g, s in zip(self.param_groups, state):
            g.update(s)
