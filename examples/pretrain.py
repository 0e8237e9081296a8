#!/usr/bin/env python
"""Pre-train a Llama- or GPT-style decoder with the tiered engine.

One GPU (or CPU with the tiny presets):

    python examples/pretrain.py --model llama:tiny --steps 20
    python examples/pretrain.py --model gpt:gpt2-small --data tokens.u16 --steps 1000 \\
        --save-dir ckpt --save-every 200

Several GPUs of one node (one process per GPU):

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \\
        examples/pretrain.py --model llama:llama3-70b --flextrain-config examples/llama3_70b_8gpu.json

Without ``--flextrain-config`` the tier split is planned from the free HBM and host DRAM of the
machine (everything in HBM when it fits); the JSON file gives full control (the reference's schema).

``--data`` names a flat binary file of token ids (``.u16`` / ``.u32`` / ``.i32`` / ``.i64``, see
``flextrain_b200.data.TokenFile``); without it random tokens are used.  ``--resume DIR`` continues
from what ``--save-dir DIR`` wrote: optimizer state, loss scaler, RNG and the position in the data.
"""
import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import flextrain_b200 as flextrain  # noqa: E402
from flextrain_b200.config import init_flextrain_config  # noqa: E402
from flextrain_b200.data import MicroBatchFeeder, SyntheticTokens, TokenFile  # noqa: E402
from flextrain_b200.lr_schedule import LRSchedule  # noqa: E402
from flextrain_b200.ops.adam import FlexTrainAdam  # noqa: E402
from flextrain_b200.utils.timer import ThroughputReporter, llama_flops_per_token  # noqa: E402

DEFAULT_CONFIG = {
    "batch_size": 4, "micro_batch_size": 2, "checkpoint_interval": 1,
    "split_ratio": {"parameter": [1.0, 0.0], "optimizer": [1.0, 0.0], "checkpoint": [1.0, 0.0],
                    "gradient": [1.0, 0.0], "alpha": 0.0},
}


def build_model(spec: str, args, device, dtype):
    family, _, name = spec.partition(":")
    over = {}
    if args.layers:
        over["num_layers"] = args.layers
    if args.seq_len:
        over["seq_len"] = args.seq_len
    if family == "llama":
        from flextrain_b200.models import llama as fam
        block = fam.LlamaBlock
        model_cls = fam.LlamaModel
    elif family == "gpt":
        from flextrain_b200.models import gpt as fam
        block = fam.GPTBlock
        model_cls = fam.GPTModel
    else:
        raise SystemExit(f"unknown model family '{family}' (use llama:<preset> or gpt:<preset>)")
    if name not in fam.PRESETS:
        raise SystemExit(f"unknown {family} preset '{name}'; known: {', '.join(fam.PRESETS)}")
    cfg = fam.preset(name, **over)
    with flextrain.Init(layer_class=block, num_layers=cfg.num_layers,
                        param_grouping_func=fam.param_grouping, init_device=device):
        model = model_cls(cfg, dtype=dtype, device=device)
    return fam, cfg, model


def plan_split(args, world):
    """Tier split from the capacities of this machine: HBM first, then host DRAM, then NVMe."""
    import psutil
    from flextrain_b200 import planner
    family, _, name = args.model.partition(":")
    fam = __import__(f"flextrain_b200.models.{family}", fromlist=["preset"])
    over = {k: v for k, v in (("num_layers", args.layers), ("seq_len", args.seq_len)) if v}
    shape = planner.shape_of(fam.preset(name, **over), args.micro_batch_size)
    hbm_free, _ = torch.cuda.mem_get_info()
    budget = planner.MemoryBudget(hbm_free, psutil.virtual_memory().available / world * 0.85, 0.0)
    split = planner.plan(shape, world, args.micro_batches_per_rank, budget, unit_buffers=2)
    if split is None:
        raise SystemExit(f"{args.model} does not fit HBM + host DRAM of {world} rank(s); "
                         "pass --flextrain-config with an nvme_swap section")
    return split


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    flextrain.add_config_arguments(ap)
    ap.add_argument("--model", default="llama:tiny", help="<family>:<preset>, family llama or gpt")
    ap.add_argument("--layers", type=int, default=0, help="override the preset's layer count")
    ap.add_argument("--seq-len", type=int, default=0, help="override the preset's sequence length")
    ap.add_argument("--data", default=None, help="flat binary token file; random tokens when absent")
    ap.add_argument("--micro-batch-size", type=int, default=2, help="without --flextrain-config")
    ap.add_argument("--micro-batches-per-rank", type=int, default=2, help="without --flextrain-config")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--warmup-steps", type=int, default=0)
    ap.add_argument("--lr-decay", default="constant", choices=["constant", "cosine", "linear"])
    ap.add_argument("--total-steps", type=int, default=0, help="length of the decay (default: --steps)")
    ap.add_argument("--weight-decay", type=float, default=0.1)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--log-every", type=int, default=1)
    ap.add_argument("--eval-every", type=int, default=0, help="validation pass every N steps (0: never)")
    ap.add_argument("--eval-data", default=None, help="token file of the validation pass (default: --data)")
    ap.add_argument("--save-dir", default=None)
    ap.add_argument("--save-every", type=int, default=0, help="0: only at the end")
    ap.add_argument("--resume", default=None, help="directory written by --save-dir")
    ap.add_argument("--init-weights", default=None,
                    help="torch file of named tensors (this package's names) to start from")
    ap.add_argument("--export", default=None, help="write the final weights (named fp32 tensors) here")
    ap.add_argument("--metrics-file", default=None, help="append one JSON record per step (rank 0)")
    args = ap.parse_args()

    flextrain.init_distributed(dist_backend="nccl" if torch.cuda.is_available() else "gloo",
                               force_init=int(os.environ.get("WORLD_SIZE", "1")) > 1)
    rank, world = flextrain.distributed.get_rank(), flextrain.distributed.get_world_size()
    device = flextrain.distributed.current_device()
    cuda = device.type == "cuda"

    if args.flextrain_config:
        with open(args.flextrain_config) as f:
            ft_cfg = json.load(f)
    else:
        ft_cfg = json.loads(json.dumps(DEFAULT_CONFIG))
        ft_cfg["micro_batch_size"] = args.micro_batch_size
        ft_cfg["batch_size"] = args.micro_batch_size * args.micro_batches_per_rank * world
        if cuda:
            ft_cfg["split_ratio"] = plan_split(args, world)
    ft_cfg.setdefault("mixed_precision", {"device_dtype": "bf16" if cuda else "fp32"})
    init_flextrain_config(ft_cfg, log=rank == 0)
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[
        ft_cfg["mixed_precision"].get("device_dtype", "bf16")]

    torch.manual_seed(args.seed)
    fam, cfg, model = build_model(args.model, args, device, dtype)
    opt = FlexTrainAdam(fam.make_param_groups(model, weight_decay=args.weight_decay), lr=args.lr,
                        betas=(0.9, 0.95), eps=1e-8, weight_decay=args.weight_decay)

    source = TokenFile(args.data) if args.data else SyntheticTokens(cfg.vocab)
    mbs = ft_cfg["micro_batch_size"]
    feeder = MicroBatchFeeder(source, mbs, cfg.seq_len, device=device, rank=rank, world=world,
                              seed=args.seed)
    # validation draws from its own stream through the same callback
    eval_source = TokenFile(args.eval_data) if args.eval_data else source
    eval_feeder = MicroBatchFeeder(eval_source, mbs, cfg.seq_len, device=device, rank=rank, world=world,
                                   seed=args.seed + 1) if args.eval_every else None
    active = {"feeder": feeder}
    flextrain.set_llm_func(*fam.make_llm_funcs(model, lambda: active["feeder"]()))
    engine = flextrain.initialize(model, opt, dist_init_required=False)

    sched = LRSchedule(opt, peak_lr=args.lr, warmup_steps=args.warmup_steps,
                       total_steps=(args.total_steps or args.steps) if args.lr_decay != "constant" else None,
                       decay=args.lr_decay)
    engine.register_post_step_function(sched.step)
    start_step = 0
    if args.init_weights:
        engine.import_state_dict(torch.load(args.init_weights, map_location="cpu", mmap=True))
    if args.resume:
        engine.load(args.resume)
        with open(os.path.join(args.resume, f"rank{rank}_data.json")) as f:
            extra = json.load(f)
        feeder.load_state_dict(extra["data"])
        sched.load_state_dict(extra["lr_schedule"])
        start_step = engine.global_steps + engine.skipped_steps
        flextrain.rank0_logger.info(f"resumed from {args.resume} at step {start_step}")

    def save(directory):
        engine.save(directory)
        with open(os.path.join(directory, f"rank{rank}_data.json"), "w") as f:
            json.dump({"data": feeder.state_dict(), "lr_schedule": sched.state_dict()}, f)

    tokens_per_step = ft_cfg["batch_size"] * cfg.seq_len
    fpt = llama_flops_per_token(cfg.num_layers, cfg.hidden, cfg.ffn, cfg.vocab, cfg.seq_len,
                                cfg.num_heads, getattr(cfg, "num_kv_heads", None))
    reporter = ThroughputReporter(tokens_per_step, fpt, world)
    flextrain.rank0_logger.info(f"{args.model}: {cfg.total_numel / 1e6:.1f} M parameters, "
                                f"{tokens_per_step} tokens per step on {world} rank(s), device {device}")
    from flextrain_b200.utils.metrics import MetricsLog
    metrics = MetricsLog(args.metrics_file, engine, tokens_per_step, fpt, world) if args.metrics_file else None
    t_last, losses = time.time(), []
    for step in range(start_step, start_step + args.steps):
        lr_used = sched.current_lrs[0]
        out = engine.train_iteration()
        local = sum(float(l.detach().float()) for l in out) / len(out)       # reads the loss back
        loss = flextrain.distributed.all_reduce_scalar(local) / world
        losses.append(loss)
        if metrics is not None:
            metrics.step(None, loss=loss, lr=lr_used)
        if (step + 1) % args.log_every == 0:
            now = time.time()
            rep = reporter.report((now - t_last) / args.log_every)
            t_last = now
            flextrain.distributed.print_rank0(
                f"step {step + 1:6d}  loss {loss:8.4f}  {rep['tokens_per_s']:10.0f} tok/s  "
                f"{rep['tflops_per_gpu']:7.1f} TFLOPS/GPU  lr {lr_used:.3g}  scale {engine.loss_scale:g}")
        if eval_feeder is not None and (step + 1) % args.eval_every == 0:
            active["feeder"] = eval_feeder
            val = engine.eval_iteration()
            active["feeder"] = feeder
            val_loss = flextrain.distributed.all_reduce_scalar(sum(float(v) for v in val) / len(val)) / world
            flextrain.distributed.print_rank0(f"step {step + 1:6d}  validation loss {val_loss:8.4f}")
            t_last = time.time()
        if args.save_dir and args.save_every and (step + 1) % args.save_every == 0:
            save(args.save_dir)
    engine.synchronize()
    if args.save_dir:
        save(args.save_dir)
    if args.export:
        weights = engine.export_state_dict()           # collective; rank 0 gets the dict
        if rank == 0:
            torch.save(weights, args.export)
    if rank == 0:
        print(json.dumps({"final_loss": losses[-1] if losses else None, "first_loss": losses[0] if losses else None,
                          "steps_done": start_step + args.steps, "losses": losses}), flush=True)
    if metrics is not None:
        metrics.close()
    feeder.close()
    if eval_feeder is not None:
        eval_feeder.close()
    engine.shutdown()


if __name__ == "__main__":
    main()
