#!/usr/bin/env python
"""Where one training step's GPU time goes: kernel timeline of a single step.

    python benchmarks/step_profile.py [--model llama2-13b] [--warmup 3] [--top 20] [--gaps 12]
                                      [--json out.json]

Builds the engine exactly like ``bench.py`` (same model choice, tier split, data),
runs the warm-up steps, then records ONE step with the PyTorch profiler restricted
to device activity (kernels and copies; no Python or operator events, so the trace
stays small and the step is barely disturbed) and prints

  * the step's span on the device, the time during which at least one kernel or copy
    was running (union over streams), and the time during which the compute stream's
    kernels were running: ``span - busy`` is what the GPU spent waiting;
  * busy time per stream;
  * the kernels with the largest total duration (count, total, mean), and for each the
    median duration of the calls that ran alone and of those that overlapped work of
    another stream (copies, the optimizer's kernels);
  * the longest idle gaps of the union timeline with the work on either side.

Times from a profiled step explain a number, they are not one: quote ``bench.py``.
One GPU; for a multi-GPU run every rank would write the same kind of summary.
"""
import argparse
import json
import os
import sys
import tempfile
from collections import defaultdict

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def summarize_trace(events, top=20, gaps=12):
    """``events``: the ``traceEvents`` of a Chrome trace.  Returns a dict of the
    figures described in the module docstring (times in milliseconds)."""
    dev = [e for e in events
           if e.get("ph") == "X" and e.get("cat") in ("kernel", "gpu_memcpy", "gpu_memset") and e.get("dur", 0) > 0]
    if not dev:
        return {"kernels": 0}
    dev.sort(key=lambda e: e["ts"])
    t0 = dev[0]["ts"]
    t1 = max(e["ts"] + e["dur"] for e in dev)
    per_stream = defaultdict(float)
    by_name = defaultdict(lambda: [0, 0.0])
    for e in dev:
        per_stream[str(e.get("args", {}).get("stream", "?"))] += e["dur"]
        rec = by_name[e["name"]]
        rec[0] += 1
        rec[1] += e["dur"]
    # union of intervals, and the gaps between its pieces
    busy = 0.0
    idle = []
    cur_s, cur_e, last = dev[0]["ts"], dev[0]["ts"] + dev[0]["dur"], dev[0]
    for e in dev[1:]:
        s, en = e["ts"], e["ts"] + e["dur"]
        if s > cur_e:
            busy += cur_e - cur_s
            idle.append((s - cur_e, cur_e - t0, last["name"], e["name"]))
            cur_s, cur_e, last = s, en, e
        elif en > cur_e:
            cur_e, last = en, e
    busy += cur_e - cur_s
    idle.sort(reverse=True)
    main_stream = max(per_stream, key=per_stream.get)
    # per kernel name: durations of the calls that ran alone and of those that shared the GPU with
    # work of another stream for at least a tenth of their time
    stream_of = lambda e: str(e.get("args", {}).get("stream", "?"))   # noqa: E731
    alone, shared = defaultdict(list), defaultdict(list)
    others = [(e["ts"], e["ts"] + e["dur"], stream_of(e)) for e in dev]
    lo = 0
    for e in dev:
        s0, s1, st = e["ts"], e["ts"] + e["dur"], stream_of(e)
        while lo < len(others) and others[lo][1] < s0 - 5e5:        # nothing runs for half a second
            lo += 1
        ov = 0.0
        for a, b, ost in others[lo:]:
            if a >= s1:
                break
            if ost != st:
                ov += max(0.0, min(b, s1) - max(a, s0))
        (shared if ov > 0.1 * e["dur"] else alone)[e["name"]].append(e["dur"])
    med = lambda v: sorted(v)[len(v) // 2] if v else None             # noqa: E731
    ms = 1e-3
    short = lambda n: n if len(n) <= 90 else n[:87] + "..."          # noqa: E731
    return {
        "kernels": len(dev),
        "span_ms": (t1 - t0) * ms,
        "busy_union_ms": busy * ms,
        "idle_ms": (t1 - t0 - busy) * ms,
        "busiest_stream": main_stream,
        "per_stream_busy_ms": {k: v * ms for k, v in sorted(per_stream.items(), key=lambda kv: -kv[1])},
        "top_kernels": [{"name": short(n), "count": c, "total_ms": t * ms, "mean_us": t / c,
                         "alone": len(alone[n]), "alone_median_us": med(alone[n]),
                         "alone_min_us": min(alone[n]) if alone[n] else None,
                         "shared": len(shared[n]), "shared_median_us": med(shared[n])}
                        for n, (c, t) in sorted(by_name.items(), key=lambda kv: -kv[1][1])[:top]],
        "idle_gaps": [{"gap_us": g, "at_ms": at * ms, "after": short(a), "before": short(b)}
                      for g, at, a, b in idle[:gaps]],
        "idle_gap_count": len(idle),
        "idle_in_gaps_over_50us_ms": sum(g for g, *_ in idle if g > 50) * ms,
    }


def format_summary(s) -> str:
    if not s.get("kernels"):
        return "no device activity in the trace"
    out = [f"{s['kernels']} kernels/copies; span {s['span_ms']:.1f} ms, busy (any stream) "
           f"{s['busy_union_ms']:.1f} ms, idle {s['idle_ms']:.1f} ms "
           f"({100 * s['idle_ms'] / s['span_ms']:.1f} %), of which {s['idle_in_gaps_over_50us_ms']:.1f} ms "
           f"in gaps over 50 us ({s['idle_gap_count']} gaps)"]
    out.append("busy per stream (ms): " + ", ".join(f"{k}: {v:.1f}" for k, v in s["per_stream_busy_ms"].items()))
    out.append("top kernels by total time (calls that ran alone: count, min, median; calls that shared the GPU "
               "with another stream: count, median):")
    us = lambda v: "-" if v is None else f"{v:.0f}"                   # noqa: E731
    for k in s["top_kernels"]:
        out.append(f"  {k['total_ms']:9.2f} ms  x{k['count']:<6d} {k['mean_us']:9.1f} us  "
                   f"[alone x{k.get('alone', 0)} min {us(k.get('alone_min_us'))} med {us(k.get('alone_median_us'))} | "
                   f"shared x{k.get('shared', 0)} med {us(k.get('shared_median_us'))}]  {k['name']}")
    out.append("longest idle gaps:")
    for g in s["idle_gaps"]:
        out.append(f"  {g['gap_us']:9.1f} us at +{g['at_ms']:8.1f} ms  after [{g['after']}]  before [{g['before']}]")
    return "\n".join(out)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="auto")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--seq-len", type=int, default=0)
    ap.add_argument("--micro-batches-per-rank", type=int, default=0)
    ap.add_argument("--unit-buffers", type=int, default=3)
    ap.add_argument("--alpha", type=float, default=0.25)
    ap.add_argument("--top", type=int, default=20)
    ap.add_argument("--gaps", type=int, default=12)
    ap.add_argument("--json", default=None, help="also write the summary as JSON here")
    args = ap.parse_args()

    import psutil
    import torch
    from torch.profiler import ProfilerActivity, profile

    import bench
    import flextrain_b200 as ft
    from flextrain_b200.config import init_flextrain_config
    from flextrain_b200.models.llama import (LlamaBlock, LlamaModel, make_llm_funcs, make_param_groups,
                                             param_grouping)
    from flextrain_b200.ops.adam import FlexTrainAdam

    ft.init_distributed(dist_backend="nccl", force_init=False)
    dev = ft.distributed.current_device()
    hbm_free, _ = torch.cuda.mem_get_info()
    args.nvme_gib_per_rank = 0.0
    dram, node_gpus = psutil.virtual_memory().available, torch.cuda.device_count()
    name, _ = bench.pick_model(args, hbm_free, dram, node_gpus)
    mcfg = bench._model_cfg(name, args)
    mbs, mbpr = bench.MICRO_BATCH.get(name, 2), args.micro_batches_per_rank or 1
    split = bench.plan_split(args, name, 1, hbm_free, dram, node_gpus)
    if split is None:
        raise SystemExit(f"{name} does not fit on one GPU")
    cfg = {"batch_size": mbs * mbpr, "micro_batch_size": mbs, "checkpoint_interval": 1, "split_ratio": split,
           "mixed_precision": {"device_dtype": "bf16", "gradacc_dtype": "fp32", "master_dtype": "fp32",
                               "dynamic_loss_scaling": False, "loss_scale": 1.0},
           "nvme_swap": {"swap_dir": os.path.join(tempfile.gettempdir(), "ft_b200_swap")},
           "engine": {"num_unit_buffers": args.unit_buffers}}
    init_flextrain_config(cfg, log=True)
    torch.manual_seed(0)
    with ft.Init(layer_class=LlamaBlock, num_layers=mcfg.num_layers, param_grouping_func=param_grouping,
                 init_device=dev):
        model = LlamaModel(mcfg, dtype=torch.bfloat16, device=dev)
    opt = FlexTrainAdam(make_param_groups(model, weight_decay=0.1), lr=1e-4, betas=(0.9, 0.95), eps=1e-8,
                        weight_decay=0.1)
    gen = torch.Generator().manual_seed(1)
    pool = [torch.randint(0, mcfg.vocab, (mbs, mcfg.seq_len + 1), generator=gen).to(dev)
            for _ in range(max(2, mbpr))]
    state = {"i": 0}

    def batch_fn():
        t = pool[state["i"] % len(pool)]
        state["i"] += 1
        return t[:, :-1], t[:, 1:]

    ft.set_llm_func(*make_llm_funcs(model, batch_fn))
    engine = ft.initialize(model, opt, dist_init_required=False)
    for _ in range(args.warmup):
        engine.train_iteration()
        engine.synchronize()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        start.record()
        engine.train_iteration()
        engine.synchronize()
        end.record()
        torch.cuda.synchronize()
    trace = os.path.join(tempfile.gettempdir(), f"ft_step_trace_{os.getpid()}.json")
    prof.export_chrome_trace(trace)
    with open(trace) as f:
        events = json.load(f)["traceEvents"]
    os.unlink(trace)
    summary = summarize_trace(events, args.top, args.gaps)
    summary["model"] = name
    summary["step_ms_cuda_events_profiled"] = start.elapsed_time(end)
    print(f"{name}: profiled step {summary['step_ms_cuda_events_profiled']:.1f} ms (CUDA events)")
    print(format_summary(summary))
    if args.json:
        with open(args.json, "w") as f:
            json.dump(summary, f, indent=1)
    engine.shutdown()


if __name__ == "__main__":
    main()
