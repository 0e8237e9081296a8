#!/usr/bin/env python
"""Headline benchmark: tokens/s (and TFLOPS/GPU) of tiered-offload training of a
Llama-shape model on N GPUs of one node.

    python bench.py --gpus N --steps K --warmup W            # this engine
    python bench.py --impl reference --gpus N ...            # unmodified reference

For N > 1 launch with ``python -m torch.distributed.run --nproc-per-node N``.
Rank 0 prints ONE JSON line.  ``value`` is device-timed (CUDA events, max over
ranks) with token batches already on the device; ``e2e.value`` times the same
steps through the public API with every micro-batch copied from pinned host
memory and every loss read back to the host.

Model: the largest of llama3-70b / llama2-13b / llama2-7b whose bf16 parameters
plus fp32 master weights and Adam moments (14 bytes per parameter) fit the HBM +
host DRAM of the N ranks (``--model`` overrides).  Data: synthetic uniform
tokens; weights: N(0, 0.02) from a fixed seed.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

MICRO_BATCH = {"llama3-70b": 2, "llama2-13b": 8, "llama2-7b": 4, "tiny": 2}
METRIC = "tokens/sec & TFLOPS/GPU, Llama-70B-shape tiered offload at 1/2/4/8 B200"


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=4)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--model", default="auto")
    p.add_argument("--micro-batches-per-rank", type=int, default=0)
    p.add_argument("--seq-len", type=int, default=0)
    p.add_argument("--layers", type=int, default=0, help="debug only: truncates the model")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--unit-buffers", type=int, default=3)
    p.add_argument("--alpha", type=float, default=0.25)
    p.add_argument("--split", default="", help="JSON split_ratio override")
    p.add_argument("--engine", default="", help="JSON object merged into the config's engine section")
    p.add_argument("--phases", action="store_true",
                   help="also report the device time of forward / backward / finish of the last step")
    return p.parse_args()


# ------------------------------------------------------------------ clocks
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.path = tempfile.NamedTemporaryFile(prefix="ft_clocks_", suffix=".csv", delete=False).name
        self.proc = None
        self.gpu_index = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200", "-i", str(self.gpu_index)],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                parts = [x.strip() for x in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1]))
                    mx.append(float(parts[2]))
                    power.append(float(parts[3]))
                except ValueError:
                    continue
                for name, val in zip(names, parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        os.unlink(self.path)
        # keep the samples taken under load (the upper half by power draw)
        if sm:
            cut = statistics.median(power)
            loaded = [s for s, p in zip(sm, power) if p >= cut] or sm
            return {"sm_mhz": statistics.median(loaded), "sm_max_mhz": max(mx),
                    "power_w_max": max(power), "samples": len(sm), "reasons": sorted(reasons)}
        return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}


# ---------------------------------------------------------------- our arm
def pick_model(args, world, hbm_free, dram_avail):
    from flextrain_b200 import planner
    from flextrain_b200.models.llama import preset
    names = ["llama3-70b", "llama2-13b", "llama2-7b"] if args.model == "auto" else [args.model]
    why = {}
    for name in names:
        cfg = preset(name)
        if args.seq_len:
            cfg.seq_len = args.seq_len
        if args.layers:
            cfg.num_layers = args.layers
        mbs = MICRO_BATCH.get(name, 2)
        mbpr = args.micro_batches_per_rank or 1
        shape = planner.shape_of(cfg, mbs)
        budget = planner.MemoryBudget(hbm_free, dram_avail / world * 0.85, 0.0)
        split = planner.plan(shape, world, mbpr, budget, unit_buffers=args.unit_buffers,
                             alpha=args.alpha)
        if split is not None or args.model != "auto":
            return name, cfg, mbs, mbpr, split, why
        need = shape.total_numel * 14 / 2 ** 30
        why[name] = (f"needs {need:.0f} GiB of parameter+optimizer state; {world} rank(s) offer "
                     f"{world * hbm_free / 2 ** 30:.0f} GiB HBM + {dram_avail * 0.85 / 2 ** 30:.0f} GiB DRAM")
    raise SystemExit("no model fits")


def run_ours(args):
    import psutil
    import torch
    import flextrain_b200 as ft
    from flextrain_b200.config import init_flextrain_config
    from flextrain_b200.models.llama import (LlamaBlock, LlamaModel, make_llm_funcs,
                                             make_param_groups, param_grouping)
    from flextrain_b200.ops.adam import FlexTrainAdam
    from flextrain_b200.ops.native import cuda_lib
    from flextrain_b200.utils.timer import llama_flops_per_token

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    # A run that stops making progress dumps every thread's Python stack and exits instead
    # of sitting in the launcher until someone kills it (re-armed before every step).
    import faulthandler
    stall_init = int(os.environ.get("FLEXTRAIN_BENCH_INIT_LIMIT", "1500"))
    stall_step = int(os.environ.get("FLEXTRAIN_BENCH_STEP_LIMIT", "600"))

    def arm(seconds):
        faulthandler.cancel_dump_traceback_later()
        if seconds > 0:
            faulthandler.dump_traceback_later(seconds, exit=True)

    arm(stall_init)
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit(f"--gpus {args.gpus} needs a torch.distributed.run launch with "
                             f"--nproc-per-node {args.gpus}")
    ft.init_distributed(dist_backend="nccl", force_init=world > 1)
    dev = ft.distributed.current_device()
    lib = cuda_lib()                       # fail loudly if the native library is missing
    hbm_free, _ = torch.cuda.mem_get_info()
    dram_avail = psutil.virtual_memory().available
    name, mcfg, mbs, mbpr, split, skipped = pick_model(args, world, hbm_free, dram_avail)
    if args.split:
        split = json.loads(args.split)
    if split is None:
        raise SystemExit(f"{name} does not fit on {world} GPU(s)")
    seq = mcfg.seq_len
    cfg = {"batch_size": mbs * mbpr * world, "micro_batch_size": mbs, "checkpoint_interval": 1,
           "split_ratio": split,
           "mixed_precision": {"device_dtype": "bf16", "gradacc_dtype": "fp32", "master_dtype": "fp32",
                               "dynamic_loss_scaling": False, "loss_scale": 1.0},
           "nvme_swap": {"swap_dir": os.path.join(tempfile.gettempdir(), "ft_b200_swap")},
           "engine": {"num_unit_buffers": args.unit_buffers, "phase_timing": bool(args.phases)}}
    if args.engine:
        cfg["engine"].update(json.loads(args.engine))
    init_flextrain_config(cfg, log=rank == 0)
    t_init = time.time()
    torch.manual_seed(0)
    with ft.Init(layer_class=LlamaBlock, num_layers=mcfg.num_layers,
                 param_grouping_func=param_grouping, init_device=dev):
        model = LlamaModel(mcfg, dtype=torch.bfloat16, device=dev)
    opt = FlexTrainAdam(make_param_groups(model, weight_decay=0.1), lr=1e-4, betas=(0.9, 0.95),
                        eps=1e-8, weight_decay=0.1)

    # synthetic data: a pool of pinned host batches and a device-resident copy
    gen = torch.Generator().manual_seed(1 + rank)
    pool = [torch.randint(0, mcfg.vocab, (mbs, seq + 1), generator=gen).pin_memory()
            for _ in range(max(2, mbpr))]
    dev_pool = [t.to(dev) for t in pool]
    state = {"i": 0, "host": False, "h2d": 0}

    def batch_fn():
        i = state["i"] % len(pool)
        state["i"] += 1
        if state["host"]:
            t = pool[i].to(dev, non_blocking=True)
            state["h2d"] += pool[i].numel() * pool[i].element_size()
        else:
            t = dev_pool[i]
        return t[:, :-1], t[:, 1:]

    ft.set_llm_func(*make_llm_funcs(model, batch_fn))
    engine = ft.initialize(model, opt, dist_init_required=False)
    torch.cuda.synchronize()
    init_s = time.time() - t_init

    def barrier():
        ft.distributed.barrier()
        torch.cuda.synchronize()

    def timed(steps, read_loss):
        barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        d2h = 0
        last = None
        for _ in range(steps):
            arm(stall_step)
            losses = engine.train_iteration()
            if read_loss:
                last = [float(l.detach().float().item()) for l in losses]
                d2h += 4 * len(losses)
        engine.synchronize()
        end.record()
        barrier()
        ms = start.elapsed_time(end)
        ms = ft.distributed.all_reduce_scalar(ms, ft.distributed.ReduceOp.MAX)
        return ms / steps, d2h / max(steps, 1), last

    def note(msg):
        # progress lines on stderr (rank 0): a run that stalls shows how far it got
        if rank == 0:
            print(f"[bench +{time.time() - t_init:7.1f}s] {msg}", file=sys.stderr, flush=True)

    note(f"engine ready, {args.warmup} warm-up steps follow")
    for i in range(args.warmup):
        arm(stall_step)
        t_w = time.time()
        engine.train_iteration()
        engine.synchronize()
        note(f"warm-up step {i + 1} took {time.time() - t_w:.2f} s (host wall, synchronised)")

    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0"))) if rank == 0 else None
    launches0 = lib.ft_launch_count() if hasattr(lib, "ft_launch_count") else 0
    if sampler:
        sampler.start()
    note("timed steps (device-timed region) begin")
    ms_dev, _, _ = timed(args.steps, read_loss=False)
    note(f"timed region done: {ms_dev:.1f} ms/step")
    launches = (lib.ft_launch_count() - launches0) if hasattr(lib, "ft_launch_count") else None
    clocks = sampler.stop() if sampler else None

    e2e = None
    if not args.no_e2e:
        state["host"], state["h2d"] = True, 0
        ms_e2e, d2h_per_step, last_loss = timed(args.steps, read_loss=True)
        tokens = mbs * mbpr * world * seq
        e2e = {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e,
               "h2d_bytes_per_step": state["h2d"] // args.steps, "d2h_bytes_per_step": int(d2h_per_step),
               "last_loss": last_loss}
    tokens = mbs * mbpr * world * seq
    tps = tokens / (ms_dev / 1e3)
    fpt = llama_flops_per_token(mcfg.num_layers, mcfg.hidden, mcfg.ffn, mcfg.vocab, seq,
                                mcfg.num_heads, mcfg.num_kv_heads, recompute=False)
    arm(stall_step)
    health = engine.health()
    phase_ms = engine.stats()["phase_ms"] if args.phases else None
    traffic = engine.stats()["traffic_bytes"]
    engine.shutdown()
    if rank == 0:
        out = {"metric": METRIC, "value": tps, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
               "warmup": args.warmup, "ms_per_step": ms_dev, "higher_is_better": True,
               "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
               "impl": "ours",
               "tflops_per_gpu": tps * fpt / world / 1e12,
               "config": {"model": name + (f"-{args.layers}L-DEBUG" if args.layers else ""),
                          "global_batch": mbs * mbpr * world, "micro_batch": mbs,
                          "micro_batches_per_rank": mbpr, "seq_len": seq,
                          "parallelism": f"zero3-dp{world}", "split_ratio": split,
                          "l2": "inputs and weights per step exceed L2 (126 MB) many times over",
                          "flops": "model FLOPs, 6*N*tokens + attention, recompute not counted",
                          "engine_overrides": json.loads(args.engine) if args.engine else None,
                          "larger_models_skipped": skipped,
                          "across_n": "the model is the largest that fits N ranks, so tokens/s at different N "
                                      "may refer to different models: compare tflops_per_gpu"},
               "clocks": clocks, "e2e": e2e, "gpu_launches": launches,
               "init_seconds": init_s, "skipped_steps": health["skipped_steps"],
               "error_words": {"gemm": health.get("gemm_error_word"), "comm": health.get("comm_error_word")}}
        if phase_ms is not None:
            out["phase_ms_last_step"] = phase_ms
            out["traffic_bytes_total"] = traffic
        print(json.dumps(out), flush=True)
    arm(0)


# ---------------------------------------------------------- reference arm
def run_reference(args):
    try:
        from baseline import run_reference as ref
    except Exception as exc:                                  # pragma: no cover
        print(json.dumps({"impl": "reference",
                          "unavailable": f"reference harness failed to import: {exc}"}), flush=True)
        return
    ref.main(args, METRIC, MICRO_BATCH)


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
