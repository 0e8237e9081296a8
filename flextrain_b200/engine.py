"""Step driver: runs the user's pre / layer / post callbacks unit by unit and
micro-batch by micro-batch in greedy-snake order, with recompute in backward.

Parity: flextrain/engine.py:1-406 - ``_conduct_first_unit`` :116-143,
``_conduct_forward`` :145-209, ``_conduct_last_unit`` :211-258,
``_conduct_backward`` :260-324, ``train_iteration`` :368-406, loss-scale
accessors :326-343, ``step`` no-op :345-346, post-step hooks :348-349.

What differs from the reference
  * stream ordering uses events only; there is no device-wide synchronise per
    micro-batch (flextrain/engine.py:174,288);
  * gradients really are unscaled, checked for inf/nan and the loss scaler is
    updated once per step (the reference never calls ``update_scale``);
  * ``every_layer`` may be empty (flextrain/engine.py:313 slices with ``[:-0]``);
  * throughput, per-tier traffic and health words are reported.
"""
from __future__ import annotations

import time
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch

from .checkpointing import (FWDContext, RNGStatePack, checkpointed_backward, detach_variable,
                            retrieve_tensor)
from .config import get_flextrain_config
from .llm_func import LLMFunc, retrieve_llm_loss
from .loss_scaler import create_loss_scaler
from .memory.coordinator.interlayer import get_interlayer_coordinator
from .memory.coordinator.optimizer import get_opts_coordinator
from .memory.coordinator.parameter import get_para_coordinator
from .scheduler import GreedySnakeBlockScheduler, LLMTask
from .utils import distributed as dist
from .utils.device import get_streams
from .utils.logging import logger, rank0_logger
from .utils.health import FusedCollectiveTimeout, Heartbeat, PeerFailure, StepWatchdog
from .utils.timer import StepTimer


def _split_passed_down(passed_down) -> Tuple[torch.Tensor, Tuple, int]:
    """The one tensor of a passed-down tuple, the tuple with that position
    blanked, and the position."""
    if torch.is_tensor(passed_down):
        return passed_down, (None,), 0
    items = tuple(passed_down)
    idx = [i for i, v in enumerate(items) if torch.is_tensor(v)]
    if len(idx) != 1:
        raise ValueError("passed_down must contain exactly one tensor")
    i = idx[0]
    return items[i], items[:i] + (None,) + items[i + 1:], i


def _join_passed_down(template: Tuple, pos: int, tensor: torch.Tensor) -> Tuple:
    return template[:pos] + (tensor,) + template[pos + 1:]


class FlexTrainEngine:
    """ZeRO-3 data-parallel training of a layer-stacked model whose parameters,
    optimizer state and activation checkpoints are tiered over HBM, pinned host
    DRAM and NVMe."""

    def __init__(self, model: torch.nn.Module, optimizer):
        cfg = get_flextrain_config()
        self.config = cfg
        self.model = model
        self.optimizer = optimizer
        self.device = dist.current_device()
        self.streams = get_streams()
        self.world = dist.get_world_size()
        self.para = get_para_coordinator()
        if not self.para.is_initialized:
            raise RuntimeError("no layer was built inside flextrain.Init(...)")
        self.inter = get_interlayer_coordinator()
        self.opts = get_opts_coordinator()
        self.loss_scaler = create_loss_scaler(cfg.mixed_precision)
        self._custom_loss_scale: Optional[float] = None
        self._move_buffers()
        self.opts.initialize(optimizer, self.loss_scaler)

        self.micro_batch_per_rank = cfg.micro_batches_per_rank(self.world)
        self.micro_batch_per_batch = self.micro_batch_per_rank      # reference name
        self.num_units = self.para.num_units
        self.num_layers = self.para.num_layers
        self.interval = cfg.checkpoint_interval
        self.scheduler = GreedySnakeBlockScheduler(self.micro_batch_per_rank, self.num_units)
        self._post_step_functions: List[Callable[[], Any]] = []
        self._training = True
        self.global_steps = 0
        self.skipped_steps = 0
        self.timer = StepTimer()
        self._nvtx = bool(cfg.engine.nvtx) and self.device.type == "cuda"
        self._phase_timing = bool(cfg.engine.phase_timing) and self.device.type == "cuda"
        import os as _os
        self._trace_on = bool(_os.environ.get("FLEXTRAIN_TRACE"))
        from .memory import guard_mode
        self._guard_mode = guard_mode()
        self._phase_events = []          # [(name, event)] of the last step
        self._last_overflow = False
        self._status: Dict[str, Any] = {"last_step_seconds": None, "watchdog_tripped": False}
        self.heartbeat = Heartbeat()
        self.watchdog = StepWatchdog(cfg.engine.watchdog_seconds)
        if self.opts.deferred:
            rank0_logger.info("deferred updates: strict overflow handling / gradient clipping hold every "
                              "update until backward has ended (no overlap of updates with backward)")

    def _move_buffers(self):
        for mod in self.model.modules():
            for name, buf in list(mod.named_buffers(recurse=False)):
                if buf is not None and buf.device != self.device:
                    mod._buffers[name] = buf.to(self.device)

    # --------------------------------------------------------------- modes
    def train(self):
        self._training = True
        self.model.train()
        return self

    def eval(self):
        self._training = False
        self.model.eval()
        return self

    def step(self):
        """No-op kept for Megatron-style loops: the update happens inside
        ``train_iteration``."""
        return None

    def register_post_step_function(self, fn: Callable[[], Any]):
        self._post_step_functions.append(fn)

    @property
    def loss_scale(self) -> float:
        return self._custom_loss_scale if self._custom_loss_scale is not None \
            else self.loss_scaler.loss_scale

    def override_loss_scale(self, loss_scale: float):
        self._custom_loss_scale = float(loss_scale)
        self.loss_scaler.cur_scale = float(loss_scale)

    @property
    def dynamic_loss_scaling(self) -> bool:
        return self.loss_scaler.dynamic

    # ------------------------------------------------------- per-step state
    def _reset_context(self, n: Optional[int] = None):
        n = n or self.micro_batch_per_rank
        self._pre_inputs: List[Any] = [None] * n
        self._post_inputs: List[Any] = [None] * n
        self._loss_inputs: List[Any] = [None] * n
        self._every_layer: List[Tuple] = [()] * n
        self._pd_template: List[Tuple] = [(None,)] * n
        self._pd_pos: List[int] = [0] * n
        self._rng: Dict[Tuple[int, int], RNGStatePack] = {}
        self._loss_results: List[Any] = [None] * n

    def _layer_range(self, unit: int) -> Tuple[int, int]:
        start = unit * self.interval
        return start, min(start + self.interval, self.num_layers)

    # -------------------------------------------------------------- forward
    def _unit_function(self, unit: int, mb: int) -> Callable:
        """The function a unit runs for one micro-batch.  Unit 0 also runs
        ``pre_process`` (so its backward reaches the embedding); every other
        unit maps the incoming activation through its layers."""
        start, end = self._layer_range(unit)
        if unit == 0:
            def first_unit():
                passed_down, every_layer = LLMFunc.pre_process(self._pre_inputs[mb])
                every_layer = tuple(every_layer)
                self._every_layer[mb] = every_layer
                x, template, pos = _split_passed_down(passed_down)
                self._pd_template[mb], self._pd_pos[mb] = template, pos
                out = LLMFunc.layer_forward(start, end)(*_join_passed_down(template, pos, x),
                                                        *every_layer)
                return retrieve_tensor(out)
            return first_unit

        def other_unit(x):
            args = _join_passed_down(self._pd_template[mb], self._pd_pos[mb], x)
            out = LLMFunc.layer_forward(start, end)(*args, *self._every_layer[mb])
            return retrieve_tensor(out)
        return other_unit

    def _trace(self, what: str):
        """With the environment variable FLEXTRAIN_TRACE set: one host-side line per
        scheduling event (rank, step, seconds since the step began) on stderr, so a run
        that stops shows where every rank stood.  Costs nothing when unset."""
        if self._trace_on:
            import sys
            import time
            t0 = getattr(self, "_trace_t0", None) or time.monotonic()
            print(f"[ft-trace r{dist.get_rank()} s{self.global_steps} +{time.monotonic() - t0:8.3f}] {what}",
                  file=sys.stderr, flush=True)

    def _enter_unit(self, unit: int, prev_unit: Optional[int], next_unit: Optional[int],
                    backward: bool):
        self._trace(f"enter unit {unit} ({'bwd' if backward else 'fwd'}), prefetch {next_unit}")
        if self.global_steps == 0 and unit % 2 == 1:
            # first step only: look at the fused kernels' error words every other unit, so that a
            # systematic time-out costs a few waits, not one per unit, before NCCL takes over
            self._fused_health_check()
        if prev_unit is not None and prev_unit != unit:
            self.para.release(prev_unit, keep=True)
        self.para.acquire(unit)
        if next_unit is not None and next_unit != unit:
            self.para.submit_gather(next_unit)
        if backward:
            self.opts.pre_unit_backward(unit)

    # NVTX ranges per (phase, unit, micro-batch) when ``engine.nvtx`` is set; they cost a
    # Python call each, so they are off by default.
    def _range_push(self, phase: str, task: LLMTask):
        if self._nvtx:
            torch.cuda.nvtx.range_push(f"{phase} u{task.unit} mb{task.micro_batch}")

    def _range_pop(self):
        if self._nvtx:
            torch.cuda.nvtx.range_pop()

    def _conduct_forward(self, task: LLMTask, nxt: Optional[LLMTask]):
        self._range_push("fwd", task)
        try:
            self._conduct_forward_impl(task, nxt)
        finally:
            self._range_pop()

    def _conduct_forward_impl(self, task: LLMTask, nxt: Optional[LLMTask]):
        u, mb = task.unit, task.micro_batch
        ckpt = self.inter.ckpt
        if nxt is not None and nxt.unit > 0 and (nxt.unit, nxt.micro_batch) != (u + 1, mb):
            ckpt.prefetch((nxt.unit, nxt.micro_batch))
        fn = self._unit_function(u, mb)
        rng = RNGStatePack()
        if u == 0:
            pre, post, loss_in = LLMFunc.get_batch()
            self._pre_inputs[mb], self._post_inputs[mb], self._loss_inputs[mb] = pre, post, loss_in
            with torch.no_grad():
                out = fn()
        else:
            x = ckpt.get((u, mb))
            with torch.no_grad():
                out = fn(x)
            ckpt.done_with((u, mb))
        self._rng[(u, mb)] = rng
        consumed_next = nxt is not None and (nxt.unit, nxt.micro_batch) == (u + 1, mb)
        n = self.micro_batch_per_rank
        order_pos = self._pos_in_unit(task)
        margin = order_pos < 1 or order_pos >= n - 1
        ckpt.put((u + 1, mb), out, pin_to_dram=margin, hot=consumed_next)

    def _pos_in_unit(self, task: LLMTask) -> int:
        tasks = self.scheduler.tasks
        idx = tasks.index(task)
        return idx % self.micro_batch_per_rank

    # ------------------------------------------------------------- backward
    def _conduct_last_unit(self, task: LLMTask):
        u, mb = task.unit, task.micro_batch
        start, end = self._layer_range(u)
        scale = self.loss_scale / self.micro_batch_per_rank
        with torch.enable_grad():
            if u == 0:
                pre, post, loss_in = LLMFunc.get_batch()
                self._pre_inputs[mb], self._post_inputs[mb], self._loss_inputs[mb] = pre, post, loss_in
                out = self._unit_function(0, mb)()
                x = None
            else:
                x = detach_variable(self.inter.ckpt.get((u, mb)))
                out = self._unit_function(u, mb)(x)
            passed = _join_passed_down(self._pd_template[mb], self._pd_pos[mb], out)
            outputs = LLMFunc.post_process(passed, self._post_inputs[mb])
            loss_rst = LLMFunc.loss(outputs, self._loss_inputs[mb])
            self._loss_results[mb] = loss_rst
            loss = retrieve_llm_loss(loss_rst).float() * scale
            torch.autograd.backward(loss)
        return None if x is None else x.grad

    def _conduct_backward(self, task: LLMTask, nxt: Optional[LLMTask]):
        self._range_push("bwd", task)
        try:
            self._conduct_backward_impl(task, nxt)
        finally:
            self._range_pop()

    def _conduct_backward_impl(self, task: LLMTask, nxt: Optional[LLMTask]):
        u, mb = task.unit, task.micro_batch
        ckpt, grads = self.inter.ckpt, self.inter.grad
        if nxt is not None:
            if nxt.unit > 0:
                ckpt.prefetch((nxt.unit, nxt.micro_batch))
            if nxt.micro_batch != mb:
                grads.prefetch(nxt.micro_batch)
        if u == self.num_units - 1:
            dx = self._conduct_last_unit(task)
        else:
            fn = self._unit_function(u, mb)
            dy = grads.get(mb)
            if u == 0:
                ctx = FWDContext(fn, self._rng[(u, mb)], ())
                checkpointed_backward(ctx, dy)
                dx = None
            else:
                x = ckpt.get((u, mb))
                ctx = FWDContext(fn, self._rng[(u, mb)], (x,))
                dx = checkpointed_backward(ctx, dy)[0]
            grads.done_with(mb)
        if u > 0:
            ckpt.done_with((u, mb), drop=True)
            hot = nxt is not None and nxt.micro_batch == mb and nxt.unit == u - 1
            grads.put(mb, dx, hot=hot, store=not hot)
        else:
            grads.drop(mb)
        self.opts.post_micro_batch_backward(u)

    # ------------------------------------------------------------ iteration
    def train_iteration(self):
        """One optimizer step over ``batch_size`` samples.  Returns the list of
        per-micro-batch loss results (whatever the ``loss`` callback returned)."""
        cfg = self.config
        # learn of a failed peer on the host, before anything is launched for this step
        self.heartbeat.check_peers()
        self.heartbeat.beat(self.global_steps)
        self.watchdog.step_started()
        try:
            if self.global_steps == 0:
                self._set_fused_wait(first_step=True)
            result = self._train_iteration(cfg)
            if self.global_steps == 1:
                self._set_fused_wait(first_step=False)
            if self._guard_mode:
                self.check_guards()
            return result
        except (PeerFailure, FusedCollectiveTimeout):
            raise
        except BaseException as exc:
            self.heartbeat.post_failure(f"{type(exc).__name__}: {exc}")
            failed = {r: m for r, m in self.heartbeat.failures().items() if r != dist.get_rank()}
            if failed and not isinstance(exc, KeyboardInterrupt):
                raise PeerFailure("; ".join(f"rank {r} failed: {m}" for r, m in sorted(failed.items()))) \
                    from exc
            raise
        finally:
            self.watchdog.step_finished()

    def _train_iteration(self, cfg):
        self.timer.start_step()
        self._reset_context()
        self._phase_events = []
        if self._trace_on:
            import time
            self._trace_t0 = time.monotonic()
            self._trace("step begins")
        self._mark_phase("start")
        self.opts.prune_pending()
        fwd, bwd = self.scheduler.forward_tasks, self.scheduler.backward_tasks
        self.para.submit_gather(fwd[0].unit if fwd else bwd[0].unit)

        prev_unit = None
        for i, task in enumerate(fwd):
            nxt = fwd[i + 1] if i + 1 < len(fwd) else bwd[0]
            if task.unit != prev_unit:
                following = task.unit + 1 if task.unit + 1 < self.num_units else None
                self._enter_unit(task.unit, prev_unit, following, backward=False)
                prev_unit = task.unit
            self._conduct_forward(task, nxt)

        self._mark_phase("forward")
        self._trace("forward launched")
        self.optimizer.update_states()
        for i, task in enumerate(bwd):
            nxt = bwd[i + 1] if i + 1 < len(bwd) else None
            if task.unit != prev_unit or i == 0:
                following = task.unit - 1 if task.unit > 0 else None
                self._enter_unit(task.unit, prev_unit, following, backward=True)
                prev_unit = task.unit
            self._conduct_backward(task, nxt)
            if nxt is None or nxt.unit != task.unit:
                self.opts.post_unit_backward(task.unit)
        self.para.release(prev_unit)
        self._mark_phase("backward")
        self._trace("backward launched")

        overflow = self._finish_step()
        # every step: a cross-GPU wait of the fused kernels that ran out must never pass unnoticed
        self._fused_health_check(end_of_step=True)
        self._mark_phase("finish")
        self._trace("finish launched")
        self.global_steps += 1
        if overflow:
            self.skipped_steps += 1
        for fn in self._post_step_functions:
            fn()
        self.timer.end_step()
        if cfg.auto_config and self.global_steps == 1:
            from .auto_config import system_auto_config
            system_auto_config(self)
        return list(self._loss_results)

    @torch.no_grad()
    def eval_iteration(self, micro_batches: Optional[int] = None):
        """Forward-only pass (validation): ``micro_batches`` micro-batches per rank
        (default: as many as a training step) are drawn from ``get_batch`` and run
        through every unit with the model in eval mode; returns the list of loss
        results.  Nothing is checkpointed, no gradient exists and no state changes:
        each unit is gathered once, all micro-batches pass through it, and the
        activations between units stay on the compute device.  All ranks call it
        together (the gathers are collective).  The reference has ``eval()`` but
        no forward-only iteration (flextrain/engine.py:362-366)."""
        n = micro_batches or self.micro_batch_per_rank
        was_training = self._training
        self.eval()
        try:
            self.opts.prune_pending()
            self._reset_context(n)
            acts: List[Any] = [None] * n
            last = self.num_units - 1
            self.para.submit_gather(0)
            prev_unit = None
            for u in range(self.num_units):
                self._enter_unit(u, prev_unit, u + 1 if u < last else None, backward=False)
                prev_unit = u
                for mb in range(n):
                    if u == 0:
                        pre, post, loss_in = LLMFunc.get_batch()
                        self._pre_inputs[mb], self._post_inputs[mb], self._loss_inputs[mb] = pre, post, loss_in
                        acts[mb] = self._unit_function(0, mb)()
                    else:
                        acts[mb] = self._unit_function(u, mb)(acts[mb])
                    if u == last:
                        passed = _join_passed_down(self._pd_template[mb], self._pd_pos[mb], acts[mb])
                        outputs = LLMFunc.post_process(passed, self._post_inputs[mb])
                        self._loss_results[mb] = LLMFunc.loss(outputs, self._loss_inputs[mb])
                        acts[mb] = None
            self.para.release(prev_unit)
            return list(self._loss_results)
        finally:
            if was_training:
                self.train()

    def _mark_phase(self, name: str):
        """With ``engine.phase_timing``: record an event on the compute stream at a
        phase boundary (``stats()`` turns consecutive pairs into milliseconds)."""
        if self._phase_timing:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(torch.cuda.current_stream())
            self._phase_events.append((name, ev))

    def phase_times_ms(self) -> Dict[str, float]:
        """Device time of the last step's phases on the compute stream: forward,
        backward (recompute included) and finish (waits for the optimizer stream
        and the host updates that the step needs, non-layerwise update)."""
        if len(self._phase_events) < 2:
            return {}
        self._phase_events[-1][1].synchronize()
        out = {}
        for (_, a), (name, b) in zip(self._phase_events[:-1], self._phase_events[1:]):
            out[name] = a.elapsed_time(b)
        return out

    def _finish_step(self) -> bool:
        grad_scale = 1.0 / float(self.loss_scale)
        if self.opts.deferred:
            # one verdict and one clip coefficient for the whole step, then every update
            self.optimizer.reduce_gradients()
            overflow, coef = self.opts.resolve_deferred(self.optimizer.gradient_sumsq(grad_scale))
            if overflow:
                self.optimizer.discard_gradients()
            else:
                self.optimizer.apply_update(grad_scale * coef)
            self.loss_scaler.update_scale(overflow)
            if self._custom_loss_scale is not None:
                self._custom_loss_scale = self.loss_scaler.loss_scale
            self._last_overflow = overflow
            return overflow
        overflow = self.opts.finish_step()
        overflow |= self.optimizer.step(grad_scale=grad_scale,
                                        check_overflow=self.opts.check_overflow)
        if self.opts.check_overflow:
            if self.world > 1:
                overflow = dist.all_reduce_scalar(float(overflow), dist.ReduceOp.MAX) > 0
            self.loss_scaler.update_scale(overflow)
            if self._custom_loss_scale is not None:
                self._custom_loss_scale = self.loss_scaler.loss_scale
        self._last_overflow = overflow
        return overflow

    # --------------------------------------------------------------- extras
    def synchronize(self):
        """Wait for every queued device and host task of this rank."""
        self.opts.wait_all()
        self.streams.synchronize()

    def stats(self, reset: bool = False) -> Dict[str, Any]:
        """Observability snapshot: bytes moved between tiers and over the fabric
        since the last reset (host-side counters), allocation totals per tier,
        step count and the last step's host wall time."""
        from .memory import TRAFFIC, allocated_bytes
        return {"traffic_bytes": TRAFFIC.snapshot(reset=reset), "allocated_bytes": allocated_bytes(),
                "global_steps": self.global_steps, "skipped_steps": self.skipped_steps,
                "last_step_seconds": self.timer.last, "phase_ms": self.phase_times_ms()}

    # bounded waits of the peer-memory kernels that ran out: start / end barriers of the
    # reduce kernels (101, 102) and of the gather (201 .. 204, and 15: a GEMM producer waiting for
    # rows that never arrived; reported in the GEMM error word)
    _COMM_TIMEOUTS = (101, 102)
    _GATHER_TIMEOUTS = (15, 201, 202, 203, 204)

    def _set_fused_wait(self, first_step: bool):
        """Wait limit of the fused kernels: longer during the first step, whose one-off
        allocations and module loads let ranks drift apart further than they ever do later."""
        if self.device.type != "cuda" or self.world == 1 or not (self.opts._fused or self.para._peer_gather):
            return
        from .parallel import fused
        steady, first = self.config.engine.fused_wait_seconds
        fused.set_wait_seconds(first if first_step else steady, self.device)

    def _fused_health_check(self, read_words=None, end_of_step: bool = False):
        """On more than one GPU, at the end of every step (and every other unit of the first
        one): if a cross-GPU wait of the fused collective kernels ran out on any rank, all
        ranks switch to the NCCL collectives for the rest of the run, the step counts as
        skipped, and - unless ``engine.fused_timeout_action`` is ``"fallback"`` -
        ``FusedCollectiveTimeout`` is raised: the kernels of a rank that gave up wrote nothing
        (its shard of the unit was not updated, a gather left the previous contents in place),
        so what the step computed cannot be trusted and the caller should reload a checkpoint.
        Costs one wait for the optimizer stream and a scalar all-reduce per step.
        ``read_words`` (tests) replaces the device error words by ``() -> (gather, reduce)``."""
        if read_words is None:
            if self.device.type != "cuda" or self.world == 1:
                return
            if not (self.opts._fused or self.para._peer_gather or self.optimizer.fused_nonlayer_in_use()):
                return
            from .ops.native import cuda_lib
            lib = cuda_lib()
            if end_of_step:
                self.streams.opt.synchronize()      # the last units' reductions have ended
            read_words = lambda: (lib.ft_gemm_error(), lib.ft_comm_error())     # noqa: E731
        gemm_word, comm_word = read_words()
        if gemm_word and gemm_word not in self._GATHER_TIMEOUTS:
            self._status["gemm_error_word_seen"] = gemm_word     # reading cleared it: keep it visible
        bad = comm_word in self._COMM_TIMEOUTS or gemm_word in self._GATHER_TIMEOUTS
        bad = dist.all_reduce_scalar(1.0 if bad else 0.0, dist.ReduceOp.MAX) > 0
        if bad:
            logger.error(f"rank {dist.get_rank()}: a bounded wait of the fused collective kernels ran out "
                         f"(error words: gather {gemm_word}, reduce {comm_word}); switching to NCCL collectives")
            self.opts._fused = False
            self.para._peer_gather = False
            self.optimizer.disable_fused_nonlayer()
            self._status["fused_collectives_disabled"] = True
            self._status["fused_timeout_words"] = {"gather": gemm_word, "reduce": comm_word,
                                                   "step": self.global_steps}
            if end_of_step:
                self.skipped_steps += 1
                if self.config.engine.fused_timeout_action == "raise":
                    self.global_steps += 1
                    raise FusedCollectiveTimeout(
                        f"step {self.global_steps - 1}: a rank waited longer than its limit for a peer inside a "
                        f"fused collective kernel (error words: gather {gemm_word}, reduce {comm_word}); "
                        "that rank's share of the step was not applied.  The run continues on the NCCL "
                        "collectives if this exception is caught; reload a checkpoint to discard the step.")

    def collectives_in_use(self) -> Dict[str, Any]:
        """Which implementation currently serves each collective of a step."""
        fused_on = self.world > 1 and self.device.type == "cuda"
        return {
            "unit_gather": "ft_peer_gather (peer loads over NVLink)" if fused_on and self.para._peer_gather
            else ("none (single rank)" if self.world == 1 else "all_gather_into_tensor"),
            "unit_reduce": "ft_rs_adam (peer reduce-scatter + unscale + Adam)" if fused_on and self.opts._fused
            else ("none (single rank)" if self.world == 1 else "reduce_scatter_tensor"),
            "non_layerwise": "ft_ar_adam (peer all-reduce + sharded Adam)"
            if fused_on and self.optimizer.fused_nonlayer_in_use()
            else ("none (single rank)" if self.world == 1 else "all_reduce"),
            "first_gemm": self.para.fused_first_gemm_state() if hasattr(self.para, "fused_first_gemm_state")
            else "separate",
            "fused_blocks": self.config.engine.fused_blocks if fused_on else None,
        }

    def check_guards(self) -> None:
        """Guard mode (FLEXTRAIN_GUARD=1): wait for all work in flight, then raise if anything
        was written next to one of the runtime's buffers (``memory.check_guards``).  Runs after
        every step in that mode; a no-op otherwise."""
        from .memory import check_guards
        self.synchronize()
        check_guards()

    def health(self) -> Dict[str, Any]:
        """Status words of the runtime: pending host updates, traffic counters,
        skipped steps, last step time, watchdog."""
        out = dict(self._status)
        out.update(global_steps=self.global_steps, skipped_steps=self.skipped_steps,
                   loss_scale=self.loss_scale, last_overflow=self._last_overflow,
                   pending_host_updates=len(self.opts._pending),
                   traffic=self.inter.traffic(), opt_d2h_bytes=self.opts.bytes_d2h)
        out.update(self.timer.summary())
        out["watchdog_tripped"] = self.watchdog.tripped
        if self.device.type == "cuda":
            from .ops.native import cuda_lib
            lib = cuda_lib()
            out["gemm_error_word"] = lib.ft_gemm_error()
            out["comm_error_word"] = lib.ft_comm_error() if hasattr(lib, "ft_comm_error") else 0
        return out

    # ------------------------------------------------------ save / resume
    def save(self, directory: str):
        """Write this rank's training state to ``directory``: ``rank{r}_unit{u}.pt`` with the
        fp32 master weights and optimizer states of every unit shard (whatever tier they
        live in) and ``rank{r}_state.pt`` with the non-layerwise parameters' state, the
        param groups' hyper-parameters and step counters, the loss scaler and the RNG
        state.  The reference has no persistent checkpoint at all (its only on-disk
        artefacts are transient swap files)."""
        import os
        self.synchronize()
        os.makedirs(directory, exist_ok=True)
        rank = dist.get_rank()
        # one file per unit, written as its states are read out of their tiers: the host never
        # holds more than one unit's fp32 master weights and moments at a time
        for u in range(self.num_units):
            torch.save(self.opts.read_states(u), os.path.join(directory, f"rank{rank}_unit{u}.pt"))
        state = {
            "world_size": self.world, "rank": rank, "global_steps": self.global_steps,
            "skipped_steps": self.skipped_steps, "num_units": self.num_units,
            "shard_numel": self.para.shard_numel, "unit_numel": self.para.unit_numel,
            "unit_files": True, "state_kinds": self.opts.K,
            "non_layerwise": self.optimizer.non_layerwise_state(),
            "param_groups": self.optimizer.hyper_state(),
            "loss_scaler": self.loss_scaler.state_dict(),
            "rng_cpu": torch.get_rng_state(),
            "rng_cuda": torch.cuda.get_rng_state() if self.device.type == "cuda" else None,
        }
        path = os.path.join(directory, f"rank{rank}_state.pt")
        torch.save(state, path)
        dist.barrier()
        return path

    @staticmethod
    def _unit_states(directory: str, head: Dict[str, Any], rank: int, unit: int, mmap: bool):
        """(master, moments...) of one unit of one rank's checkpoint: its own file, or - in
        checkpoints written before units had files of their own - an entry of the rank's state."""
        import os
        if head.get("unit_files"):
            return torch.load(os.path.join(directory, f"rank{rank}_unit{unit}.pt"), map_location="cpu",
                              weights_only=False, mmap=mmap)
        return head["units"][unit]

    def load(self, directory: str):
        """Restore what ``save`` wrote.  With the world size and partition geometry
        of the checkpoint this rank reads its own file; otherwise (a run restarted
        on fewer or more GPUs, e.g. after losing one) the shards are re-cut: every
        rank assembles its new shard of each unit from the old ranks' files that
        overlap it (read through ``mmap``, so only those pieces are touched).  RNG
        states belong to the old ranks and are then left alone."""
        import os
        self.synchronize()
        own = os.path.join(directory, f"rank{dist.get_rank()}_state.pt")
        first = os.path.join(directory, "rank0_state.pt")
        head = torch.load(first, map_location="cpu", weights_only=False, mmap=True)
        if head["num_units"] != self.num_units:
            raise ValueError("checkpoint was written for a different model partition "
                             f"({head['num_units']} units, this run has {self.num_units})")
        same = head["world_size"] == self.world and head["shard_numel"] == self.para.shard_numel
        if same:
            state = torch.load(own, map_location="cpu", weights_only=False)
            for u in range(self.num_units):
                self.opts.write_states(u, self._unit_states(directory, state, dist.get_rank(), u, mmap=False))
            self.optimizer.load_non_layerwise_state(state["non_layerwise"])
        else:
            state = head
            self._load_resharded(directory, head)
        self.optimizer.load_hyper_state(state["param_groups"])
        self.loss_scaler.load_state_dict(state["loss_scaler"])
        self.global_steps = state["global_steps"]
        self.skipped_steps = state["skipped_steps"]
        if same:
            torch.set_rng_state(state["rng_cpu"])
            if state.get("rng_cuda") is not None and self.device.type == "cuda":
                torch.cuda.set_rng_state(state["rng_cuda"])
        self.para.drain()
        self.synchronize()
        dist.barrier()

    def _load_resharded(self, directory: str, head: Dict[str, Any]):
        import os
        old_world, old_shard = head["world_size"], head["shard_numel"]
        new_shard = self.para.shard_numel
        unit_numel = self.para.unit_numel
        if head.get("unit_numel", unit_numel) != unit_numel or old_world * old_shard < unit_numel:
            raise ValueError("checkpoint was written for a different model (unit size differs)")
        files: Dict[int, Any] = {0: head}

        def old(rank: int):
            if rank not in files:
                path = os.path.join(directory, f"rank{rank}_state.pt")
                if not os.path.exists(path):
                    raise FileNotFoundError(f"{path}: the checkpoint of {old_world} ranks is incomplete")
                files[rank] = torch.load(path, map_location="cpu", weights_only=False, mmap=True)
            return files[rank]

        lo, hi = dist.get_rank() * new_shard, (dist.get_rank() + 1) * new_shard
        kinds = head.get("state_kinds") or len(head["units"][0])
        for u in range(self.num_units):
            states = [torch.zeros(new_shard, dtype=torch.float32) for _ in range(kinds)]
            for r in range(lo // old_shard, min(old_world, (hi - 1) // old_shard + 1)):
                a, b = max(lo, r * old_shard), min(hi, (r + 1) * old_shard)
                src = self._unit_states(directory, old(r), r, u, mmap=True)
                for k in range(kinds):
                    states[k][a - lo:b - lo].copy_(src[k][a - r * old_shard:b - r * old_shard])
            # what lies past the unit's true size is padding in either layout
            if hi > unit_numel:
                for k in range(kinds):
                    states[k][max(0, unit_numel - lo):].zero_()
            self.opts.write_states(u, states)
        nl = head["non_layerwise"]
        if nl:
            if nl.get("sharded", False):
                total = nl["total"]
                pieces = [old(r)["non_layerwise"] for r in range(old_world)]
                master = torch.cat([p["master"] for p in pieces])[:total]
                moments = [torch.cat([p["states"][k] for p in pieces])[:total]
                           for k in range(len(nl["states"]))]
            else:
                master, moments = nl["master"], nl["states"]
            self.optimizer.load_non_layerwise_full(master, moments)
        rank0_logger.info(f"checkpoint of {old_world} rank(s) re-cut for {self.world} rank(s)")

    # ------------------------------------------------ whole-model weights
    def _param_names(self) -> Dict[int, str]:
        return {id(p): name for name, p in self.model.named_parameters()}

    @torch.no_grad()
    def export_state_dict(self, dtype: torch.dtype = torch.float32) -> Optional[Dict[str, torch.Tensor]]:
        """The model's weights by parameter name, taken from the fp32 master copies
        of every tier and rank (what a user needs to evaluate or publish a trained
        model; the reference offers no way to get weights out).  Collective: all
        ranks call it, rank 0 receives the dict (CPU tensors of ``dtype``), the
        others None.  Memory on rank 0: the whole model in ``dtype``."""
        self.synchronize()
        names = self._param_names()
        rank0 = dist.get_rank() == 0
        out: Dict[str, torch.Tensor] = {}
        comm_dev = self.device if dist.get_backend() == "nccl" else torch.device("cpu")
        S = self.para.shard_numel
        for u in range(self.num_units):
            shard = self.opts.read_states(u)[0].to(comm_dev)
            full = torch.empty(S * self.world, dtype=torch.float32, device=comm_dev)
            dist.all_gather(full, shard)
            if rank0:
                flat = full.cpu()
                grp = self.para.unit_group(u)
                for p, off, n, shape in zip(grp.paras, grp.offsets, grp.numels, grp.shapes):
                    out[names[id(p)]] = flat[off:off + n].view(shape).to(dtype).clone()
        nl = self.optimizer.non_layerwise_master_full()
        if rank0 and nl is not None:
            off = 0
            for p in self.optimizer.non_layerwise_params:
                n = p.numel()
                out[names[id(p)]] = nl[off:off + n].view(p.shape).to(dtype).clone()
                off += n
        dist.barrier()
        return out if rank0 else None

    @torch.no_grad()
    def import_state_dict(self, state_dict: Dict[str, torch.Tensor], strict: bool = True,
                          reset_moments: bool = True):
        """Overwrite the weights from named tensors (start from pre-trained weights):
        fp32 masters and 16-bit copies of every tier are rewritten; Adam moments are
        zeroed unless ``reset_moments`` is off.  Every rank passes the same dict (for
        large models load it with ``torch.load(..., mmap=True)``) and takes its own
        shard of each unit.  With ``strict`` every parameter must be present with its
        shape; otherwise missing ones keep their value."""
        self.synchronize()
        names = self._param_names()
        known = set(names.values())
        if strict:
            missing = sorted(known - set(state_dict))
            extra = sorted(set(state_dict) - known)
            if missing or extra:
                raise KeyError(f"state dict does not match the model: missing {missing[:5]}, "
                               f"unexpected {extra[:5]}")

        def fill(dst: torch.Tensor, p, shape):
            t = state_dict.get(names[id(p)])
            if t is None:
                return False
            if tuple(t.shape) != tuple(shape):
                raise ValueError(f"{names[id(p)]}: shape {tuple(t.shape)} in the state dict, "
                                 f"{tuple(shape)} in the model")
            dst.copy_(t.reshape(-1).to(torch.float32))
            return True

        S = self.para.shard_numel
        lo, hi = dist.get_rank() * S, (dist.get_rank() + 1) * S
        for u in range(self.num_units):
            states = self.opts.read_states(u)
            grp = self.para.unit_group(u)
            for p, off, n, shape in zip(grp.paras, grp.offsets, grp.numels, grp.shapes):
                a, b = max(lo, off), min(hi, off + n)
                if a >= b:
                    continue
                t = state_dict.get(names[id(p)])
                if t is None:
                    continue
                if tuple(t.shape) != tuple(shape):
                    raise ValueError(f"{names[id(p)]}: shape {tuple(t.shape)} in the state dict, "
                                     f"{tuple(shape)} in the model")
                states[0][a - lo:b - lo].copy_(t.reshape(-1)[a - off:b - off].to(torch.float32))
            if reset_moments:
                for s in states[1:]:
                    s.zero_()
            self.opts.write_states(u, states)
        if self.optimizer.non_layerwise_params:
            full = self.optimizer.non_layerwise_master_full()
            off = 0
            for p in self.optimizer.non_layerwise_params:
                n = p.numel()
                fill(full[off:off + n], p, p.shape)
                off += n
            self.optimizer.set_non_layerwise_master(full, reset_moments)
        self.para.drain()
        self.synchronize()
        dist.barrier()

    def shutdown(self):
        self.watchdog.close()
        self.opts.shutdown()
        self.optimizer.close()
        self.para.drain()
        self.para.close()
