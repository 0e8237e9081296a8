"""Capacity plan without a run: ``python -m flextrain_b200.plan_cli --model llama:llama3-70b --gpus 8
--hbm-gib 178 --dram-gib 1000 [--nvme-gib 0] [--micro-batch 2] [--micro-batches-per-rank 1]``.

Prints the tier split the closed-form planner picks for the model and machine (as the
``split_ratio`` section of a config), the bytes every tier would hold per rank, the working set
it reserves in HBM, and a ready-to-use config file with ``--emit``.  The reference's planner
needs a profiling run on the target machine first (flextrain/auto_config.py:58-88); this is the
zero-cost sibling described in ``planner.py``.
"""
from __future__ import annotations

import argparse
import json
import sys

from . import planner

GiB = float(1 << 30)


def _model(spec: str, seq_len: int, layers: int):
    family, _, name = spec.partition(":")
    if family not in ("llama", "gpt") or not name:
        raise SystemExit("--model takes llama:<preset> or gpt:<preset>")
    mod = __import__(f"flextrain_b200.models.{family}", fromlist=["preset"])
    if name not in mod.PRESETS:
        raise SystemExit(f"unknown {family} preset '{name}'; known: {', '.join(mod.PRESETS)}")
    over = {k: v for k, v in (("seq_len", seq_len), ("num_layers", layers)) if v}
    return mod.preset(name, **over)


def plan_table(cfg, gpus: int, mbs: int, mbpr: int, hbm_gib: float, dram_gib: float, nvme_gib: float,
               unit_buffers: int = 2, alpha: float = 0.25):
    shape = planner.shape_of(cfg, mbs)
    budget = planner.MemoryBudget(hbm_gib * GiB, dram_gib * GiB / gpus, nvme_gib * GiB / gpus)
    split = planner.plan(shape, gpus, mbpr, budget, unit_buffers=unit_buffers, alpha=alpha)
    shard = shape.num_layers * shape.layer_numel / gpus
    sizes = {"parameter": shard * 2.0, "optimizer": shard * 12.0,
             "checkpoint": shape.num_layers * mbpr * shape.tokens_per_micro_batch * shape.hidden * 2.0}
    out = {"model_parameters": shape.total_numel, "state_gib_total": shape.total_numel * 14 / GiB,
           "working_set_gib": planner.working_set_bytes(shape, gpus, mbpr, unit_buffers, True, 1) / GiB,
           "split_ratio": split, "per_rank_gib": None}
    if split is not None:
        tiers = {"hbm": 0.0, "dram": 0.0, "nvme": 0.0}
        rows = {}
        for kind, total in sizes.items():
            g, c = split[kind]
            rows[kind] = {"hbm": g * total / GiB, "dram": c * total / GiB, "nvme": (1 - g - c) * total / GiB}
            for t in tiers:
                tiers[t] += rows[kind][t]
        rows["total"] = tiers
        out["per_rank_gib"] = rows
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--hbm-gib", type=float, default=178.0, help="free HBM per GPU")
    ap.add_argument("--dram-gib", type=float, default=0.0, help="host DRAM of the whole node that may be pinned")
    ap.add_argument("--nvme-gib", type=float, default=0.0, help="NVMe space of the whole node")
    ap.add_argument("--micro-batch", type=int, default=2)
    ap.add_argument("--micro-batches-per-rank", type=int, default=1)
    ap.add_argument("--seq-len", type=int, default=0)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--unit-buffers", type=int, default=2)
    ap.add_argument("--emit", default=None, help="write a config JSON with the planned split here")
    args = ap.parse_args(argv)
    cfg = _model(args.model, args.seq_len, args.layers)
    table = plan_table(cfg, args.gpus, args.micro_batch, args.micro_batches_per_rank, args.hbm_gib,
                       args.dram_gib, args.nvme_gib, args.unit_buffers)
    print(json.dumps(table, indent=1))
    if table["split_ratio"] is None:
        print(f"{args.model} does not fit {args.gpus} GPU(s) with this much DRAM / NVMe", file=sys.stderr)
        return 1
    if args.emit:
        config = {"batch_size": args.micro_batch * args.micro_batches_per_rank * args.gpus,
                  "micro_batch_size": args.micro_batch, "checkpoint_interval": 1,
                  "split_ratio": table["split_ratio"],
                  "mixed_precision": {"device_dtype": "bf16", "gradacc_dtype": "fp32", "master_dtype": "fp32"},
                  "engine": {"num_unit_buffers": args.unit_buffers}}
        if args.nvme_gib > 0:
            config["nvme_swap"] = {"swap_dir": "/tmp/flextrain_swap"}
        with open(args.emit, "w") as f:
            json.dump(config, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
