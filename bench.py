#!/usr/bin/env python
"""Headline benchmark: tokens/s (and TFLOPS/GPU) of tiered-offload training of a
Llama-shape model on N GPUs of one node.

    python bench.py --gpus N --steps K --warmup W            # this engine
    python bench.py --impl reference --gpus N ...            # unmodified reference

For N > 1 launch with ``python -m torch.distributed.run --nproc-per-node N``.
Rank 0 prints ONE JSON line.  ``value`` is device-timed (CUDA events, max over
ranks) over exactly K steps with token batches already on the device;
``e2e.value`` times steps through the public API with every micro-batch copied
from pinned host memory and every loss read back to the host (K steps when they
fit the time that is left, fewer otherwise - the count is in ``e2e.steps``).

Model.  One model per NODE, the same at every N, so that tokens/s at 1/2/4/8
GPUs is one weak-scaling curve: the largest of llama3-70b / llama2-13b /
llama2-7b whose bf16 parameters plus fp32 master weights and Adam moments (14
bytes per parameter) fit ONE GPU's HBM plus one GPU's share of the node's host
memory (``--model`` overrides).  On an 8-GPU run the Llama-3-70B shape, which no
single GPU of the node can hold, is trained as well (a child process per rank
after the main measurement) and reported under ``extra.llama3_70b``.

Data: synthetic uniform tokens, a pool of 64 distinct micro-batches per rank;
weights: N(0, 0.02) from a fixed seed.

The whole command is meant to end within ``--wall-limit`` seconds (default 780):
the end-to-end pass shrinks and the extra model is skipped when time runs short.
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

T_PROCESS_START = time.time()
REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

MICRO_BATCH = {"llama3-70b": 2, "llama2-13b": 8, "llama2-7b": 4, "tiny": 2}
CANDIDATES = ("llama3-70b", "llama2-13b", "llama2-7b")
METRIC = "tokens/sec & TFLOPS/GPU, Llama-70B-shape tiered offload at 1/2/4/8 B200"
DATA_POOL = 64
# host memory a rank may plan with: its GPU's share of what the node has free, capped so that a
# one-GPU box and one GPU of an eight-GPU box end up with the same placement
DRAM_SHARE_USE = 0.85
DRAM_PER_RANK_CAP = 96 * 2 ** 30
EXTRA_MODEL = "llama3-70b"


def parse_args(argv=None):
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
    p.add_argument("--wall-limit", type=float, default=780.0,
                   help="seconds the whole command may take; optional parts shrink or are skipped")
    p.add_argument("--extra", default="auto", choices=["auto", "on", "off"],
                   help="also train the Llama-3-70B shape after the main measurement (auto: at 8 GPUs)")
    p.add_argument("--nvme-gib-per-rank", type=float, default=0.0,
                   help="NVMe capacity the planner may use per rank (0: HBM and host memory only)")
    p.add_argument("--auto-config", action="store_true",
                   help="let the engine's profiling planner (system_auto_config) choose the split after "
                        "the first warm-up step; its measurements are added to the JSON line")
    p.add_argument("--extra-model", default=EXTRA_MODEL, help=argparse.SUPPRESS)
    p.add_argument("--as-extra", action="store_true", help=argparse.SUPPRESS)
    return p.parse_args(argv)


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


# ------------------------------------------------------------ model choice
def dram_per_rank(dram_avail: float, gpus_in_node: int) -> float:
    """Host memory one rank plans with: its GPU's share of the node's free memory."""
    return min(dram_avail / max(gpus_in_node, 1) * DRAM_SHARE_USE, DRAM_PER_RANK_CAP)


def _model_cfg(name, args):
    from flextrain_b200.models.llama import preset
    cfg = preset(name)
    if args.seq_len:
        cfg.seq_len = args.seq_len
    if args.layers:
        cfg.num_layers = args.layers
    return cfg


def pick_model(args, hbm_free, dram_avail, gpus_in_node):
    """The node's benchmark model: the largest candidate that ONE GPU with its share of the
    host memory can hold (so the same model is trained at every N).  Returns
    ``(name, reasons the larger ones were skipped)``."""
    from flextrain_b200 import planner
    if args.model != "auto":
        return args.model, {}
    why = {}
    budget = planner.MemoryBudget(hbm_free, dram_per_rank(dram_avail, gpus_in_node), 0.0)
    for name in CANDIDATES:
        cfg = _model_cfg(name, args)
        shape = planner.shape_of(cfg, MICRO_BATCH.get(name, 2))
        if planner.plan(shape, 1, args.micro_batches_per_rank or 1, budget,
                        unit_buffers=args.unit_buffers, alpha=args.alpha) is not None:
            return name, why
        why[name] = (f"needs {shape.total_numel * 14 / 2 ** 30:.0f} GiB of parameter+optimizer state; one GPU "
                     f"offers {hbm_free / 2 ** 30:.0f} GiB HBM + {budget.dram_bytes / 2 ** 30:.0f} GiB of host memory")
    raise SystemExit("no model fits one GPU of this node")


def plan_split(args, name, world, hbm_free, dram_avail, gpus_in_node):
    from flextrain_b200 import planner
    cfg = _model_cfg(name, args)
    shape = planner.shape_of(cfg, MICRO_BATCH.get(name, 2))
    budget = planner.MemoryBudget(hbm_free, dram_per_rank(dram_avail, gpus_in_node),
                                  args.nvme_gib_per_rank * 2 ** 30)
    return planner.plan(shape, world, args.micro_batches_per_rank or 1, budget,
                        unit_buffers=args.unit_buffers, alpha=args.alpha)


# ---------------------------------------------------------------- our arm
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
    stall_init = int(os.environ.get("FLEXTRAIN_BENCH_INIT_LIMIT", "600"))
    stall_step = int(os.environ.get("FLEXTRAIN_BENCH_STEP_LIMIT", "240"))

    def arm(seconds):
        faulthandler.cancel_dump_traceback_later()
        if seconds > 0:
            faulthandler.dump_traceback_later(seconds, exit=True)

    def elapsed():
        return time.time() - T_PROCESS_START

    arm(stall_init)
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit(f"--gpus {args.gpus} needs a torch.distributed.run launch with "
                             f"--nproc-per-node {args.gpus}")
    ft.init_distributed(dist_backend="nccl", force_init=world > 1)
    dev = ft.distributed.current_device()
    lib = cuda_lib()                       # fail loudly if the native library is missing

    # rank 0 chooses the model and the tier split from what IT sees; every rank uses that choice
    choice = [None]
    if rank == 0:
        hbm_free, _ = torch.cuda.mem_get_info()
        dram_avail = psutil.virtual_memory().available
        node_gpus = torch.cuda.device_count()
        name, skipped = pick_model(args, hbm_free, dram_avail, node_gpus)
        split = json.loads(args.split) if args.split else \
            plan_split(args, name, world, hbm_free, dram_avail, node_gpus)
        choice = [{"name": name, "skipped": skipped, "split": split, "node_gpus": node_gpus,
                   "dram_per_rank_gib": dram_per_rank(dram_avail, node_gpus) / 2 ** 30}]
    if world > 1:
        torch.distributed.broadcast_object_list(choice, src=0)
    name, skipped, split = choice[0]["name"], choice[0]["skipped"], choice[0]["split"]
    if split is None:
        raise SystemExit(f"{name} does not fit on {world} GPU(s)")
    mcfg = _model_cfg(name, args)
    mbs = MICRO_BATCH.get(name, 2)
    mbpr = args.micro_batches_per_rank or 1
    seq = mcfg.seq_len
    cfg = {"batch_size": mbs * mbpr * world, "micro_batch_size": mbs, "checkpoint_interval": 1,
           "split_ratio": split,
           "mixed_precision": {"device_dtype": "bf16", "gradacc_dtype": "fp32", "master_dtype": "fp32",
                               "dynamic_loss_scaling": False, "loss_scale": 1.0},
           "nvme_swap": {"swap_dir": os.path.join(tempfile.gettempdir(), "ft_b200_swap")},
           "engine": {"num_unit_buffers": args.unit_buffers, "phase_timing": bool(args.phases)}}
    if args.auto_config:
        cfg["auto_config"] = True
        cfg["max_dram_usage"] = choice[0]["dram_per_rank_gib"] * 2 ** 30 / 1e9
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

    # synthetic data: a pool of distinct pinned host batches and a device-resident copy
    gen = torch.Generator().manual_seed(1 + rank)
    pool = [torch.randint(0, mcfg.vocab, (mbs, seq + 1), generator=gen).pin_memory()
            for _ in range(max(DATA_POOL, mbpr))]
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
            print(f"[bench +{elapsed():7.1f}s] {msg}", file=sys.stderr, flush=True)

    note(f"{name}: engine ready after {init_s:.1f} s, {args.warmup} warm-up steps follow")
    from flextrain_b200.utils.health import FusedCollectiveTimeout
    for i in range(args.warmup):
        arm(stall_step)
        t_w = time.time()
        try:
            engine.train_iteration()
        except FusedCollectiveTimeout as exc:
            # every rank raises together and has switched to the library collectives; the line
            # printed at the end says so (fused_collectives_disabled)
            note(f"warm-up step {i + 1}: {exc}")
        engine.synchronize()
        note(f"warm-up step {i + 1} took {time.time() - t_w:.2f} s (host wall, synchronised)")

    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0"))) if rank == 0 else None
    launches0 = lib.ft_launch_count()
    if sampler:
        sampler.start()
    note("timed steps (device-timed region) begin")
    ms_dev, _, _ = timed(args.steps, read_loss=False)
    note(f"timed region done: {ms_dev:.1f} ms/step")
    launches = lib.ft_launch_count() - launches0
    clocks = sampler.stop() if sampler else None

    tokens = mbs * mbpr * world * seq
    e2e = None
    if not args.no_e2e:
        # as many steps as the device-timed pass when the time that is left allows it (the extra
        # model, when it follows, needs its own share)
        reserve = 360.0 if _wants_extra(args, world) else 20.0
        room = args.wall_limit - elapsed() - reserve
        affordable = int(room / (ms_dev / 1e3 * 1.05)) if room > 0 else 0
        n_e2e = max(3, min(args.steps, affordable))
        n_e2e = int(ft.distributed.all_reduce_scalar(n_e2e, ft.distributed.ReduceOp.MIN))
        state["host"], state["h2d"] = True, 0
        ms_e2e, d2h_per_step, last_loss = timed(n_e2e, read_loss=True)
        e2e = {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e,
               "steps": n_e2e, "h2d_bytes_per_step": state["h2d"] // n_e2e,
               "d2h_bytes_per_step": int(d2h_per_step), "last_loss": last_loss}
        note(f"end-to-end pass done: {ms_e2e:.1f} ms/step over {n_e2e} steps")
    tps = tokens / (ms_dev / 1e3)
    fpt = llama_flops_per_token(mcfg.num_layers, mcfg.hidden, mcfg.ffn, mcfg.vocab, seq,
                                mcfg.num_heads, mcfg.num_kv_heads, recompute=False)
    arm(stall_step)
    health = engine.health()
    stats = engine.stats()
    phase_ms = stats["phase_ms"] if args.phases else None
    final_split = engine.config.split_ratio.to_dict()
    collectives = engine.collectives_in_use()
    auto_report = getattr(engine, "auto_config_report", None)
    engine.shutdown()
    out = None
    if rank == 0:
        out = {"metric": METRIC, "value": tps, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
               "warmup": args.warmup, "ms_per_step": ms_dev, "higher_is_better": True,
               "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
               "impl": "ours",
               "tflops_per_gpu": tps * fpt / world / 1e12,
               "config": {"model": name + (f"-{args.layers}L-DEBUG" if args.layers else ""),
                          "global_batch": mbs * mbpr * world, "micro_batch": mbs,
                          "micro_batches_per_rank": mbpr, "seq_len": seq,
                          "parallelism": f"zero3-dp{world}", "split_ratio": final_split,
                          "l2": "inputs and weights per step exceed L2 (126 MB) many times over",
                          "flops": "model FLOPs, 6*N*tokens + attention, recompute not counted",
                          "data_pool": f"{len(pool)} distinct micro-batches per rank",
                          "engine_overrides": json.loads(args.engine) if args.engine else None,
                          "model_choice": "one model per node, the same at every N: the largest that one GPU "
                                          "with its share of the host memory holds",
                          "larger_models_skipped": skipped,
                          "host_memory_per_rank_gib": choice[0]["dram_per_rank_gib"]},
               "clocks": clocks, "e2e": e2e, "gpu_launches": launches,
               "init_seconds": init_s, "skipped_steps": health["skipped_steps"],
               "fused_collectives_disabled": bool(health.get("fused_collectives_disabled", False)),
               "fused_blocks": collectives.get("fused_blocks"), "collectives": collectives,
               "error_words": {"gemm": health.get("gemm_error_word"), "comm": health.get("comm_error_word")}}
        if phase_ms is not None:
            out["phase_ms_last_step"] = phase_ms
            out["traffic_bytes_total"] = stats["traffic_bytes"]
        if auto_report is not None:
            out["auto_config"] = auto_report
    arm(0)
    return out, elapsed


def _wants_extra(args, world):
    if args.as_extra or args.extra == "off":
        return False
    if args.extra == "on":
        return True
    return args.model == "auto" and world == 8


def run_extra(args, world, rank, elapsed):
    """Train the Llama-3-70B shape on the same ranks in child processes (one per rank, a
    process group of their own) and return its result for the ``extra`` key.  The parent
    has released its GPU memory and its process group; a child that does not finish within
    the time that is left is killed by its parent, so the main result is printed either way."""
    room = args.wall_limit - elapsed() - 15.0
    if room < 240.0:
        return {"unavailable": f"only {room:.0f} s of the {args.wall_limit:.0f} s limit were left"}
    env = dict(os.environ)
    env["MASTER_PORT"] = str(int(env.get("MASTER_PORT", "29500")) + 23)
    env.pop("TORCHELASTIC_USE_AGENT_STORE", None)     # the children rendezvous among themselves
    cmd = [sys.executable, os.path.abspath(__file__), "--as-extra", "--model", args.extra_model,
           "--gpus", str(world), "--steps", "4", "--warmup", "3", "--no-e2e", "--extra", "off",
           "--unit-buffers", str(args.unit_buffers), "--wall-limit", str(room)]
    if args.phases:
        cmd.append("--phases")
    if args.engine:
        cmd += ["--engine", args.engine]
    proc = subprocess.Popen(cmd, env=env, stdout=subprocess.PIPE if rank == 0 else subprocess.DEVNULL,
                            stderr=None, start_new_session=True)
    try:
        stdout, _ = proc.communicate(timeout=room)
    except subprocess.TimeoutExpired:
        os.killpg(proc.pid, 9)
        proc.wait()
        return {"unavailable": f"did not finish within the {room:.0f} s that were left"}
    if rank != 0:
        return None
    line = None
    for text in (stdout or b"").decode(errors="replace").splitlines():
        if text.startswith("{"):
            line = text
    if proc.returncode != 0 or line is None:
        return {"unavailable": f"child exited with code {proc.returncode}"}
    r = json.loads(line)
    keep = ("value", "unit", "ms_per_step", "tflops_per_gpu", "steps", "warmup", "n_gpus", "init_seconds",
            "fused_collectives_disabled", "collectives", "error_words", "gpu_launches", "phase_ms_last_step")
    res = {k: r[k] for k in keep if k in r}
    res["config"] = {k: r["config"][k] for k in ("model", "global_batch", "micro_batch", "seq_len",
                                                  "parallelism", "split_ratio")}
    return res


def main_ours(args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    out, elapsed = run_ours(args)
    if _wants_extra(args, world):
        # give everything back before the children start: GPU memory, peer mappings, process group
        import gc
        import torch
        from flextrain_b200.testing import reset_runtime
        reset_runtime()
        gc.collect()
        torch.cuda.empty_cache()
        extra = run_extra(args, world, rank, elapsed)
        if out is not None:
            out["extra"] = {args.extra_model.replace("-", "_"): extra}
    if out is not None:
        print(json.dumps(out), flush=True)


# ---------------------------------------------------------- reference arm
def run_reference(args):
    try:
        from baseline import run_reference as ref
    except Exception as exc:                                  # pragma: no cover
        print(json.dumps({"impl": "reference",
                          "unavailable": f"reference harness failed to import: {exc}"}), flush=True)
        return
    ref.main(args, METRIC, MICRO_BATCH, {"dram_share_use": DRAM_SHARE_USE,
                                         "dram_per_rank_cap": DRAM_PER_RANK_CAP})


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        main_ours(args)


if __name__ == "__main__":
    main()
