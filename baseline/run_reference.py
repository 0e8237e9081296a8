"""Reference arm of bench.py: trains the benchmark model with the UNMODIFIED
reference package from ``baseline/_ref`` through its own public API
(``Init`` / ``FlexTrainAdam`` / ``set_llm_func`` / ``initialize`` /
``engine.train_iteration``) and prints the same JSON line as the other arm.

Constraints of the reference that shape its config (all are its own asserts or
defects, none is patched): parameters and optimizer state cannot live in HBM
(GPU share asserted to 0), the NVMe tier needs libaio which this image lacks
(so every tier is host DRAM), and its fused Adam writes fp16 bit patterns
whatever the device dtype, so it runs in fp16 with its default loss scaling.
"""
from __future__ import annotations

import json
import os
import statistics
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
T_START = time.time()


def _unavailable(why: str):
    print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)


def main(args, metric, micro_batch_table, policy=None):
    """``policy``: the model-choice constants of the other arm (``dram_share_use``,
    ``dram_per_rank_cap``), so that both arms pick the same model on the same box."""
    policy = policy or {"dram_share_use": 0.85, "dram_per_rank_cap": 96 * 2 ** 30}
    ref_root = os.path.join(HERE, "_ref")
    if not os.path.isdir(os.path.join(ref_root, "flextrain")):
        return _unavailable("reference is not installed under baseline/_ref")
    # the reference and its stand-in dependency come first; this repository's package is not used
    sys.path.insert(0, os.path.join(HERE, "shims"))
    sys.path.insert(0, ref_root)
    try:
        import torch
        import flextrain
        from flextrain.config import init_flextrain_config
        from flextrain.ops.adam import FlexTrainAdam
    except Exception as exc:
        return _unavailable(f"import of the reference failed: {type(exc).__name__}: {exc}")
    import psutil
    from baseline.llama_torch import SHAPES, Block, Llama

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    try:
        if world > 1:
            flextrain.init_distributed(dist_backend="nccl")
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dev = torch.device("cuda", torch.cuda.current_device())
        name = args.model
        if name == "auto":
            name = _auto_model(torch.cuda.device_count(), torch, psutil, SHAPES, micro_batch_table, args,
                               policy)
        shape = dict(SHAPES[name])
        if args.seq_len:
            shape["seq_len"] = args.seq_len
        if args.layers:
            shape["num_layers"] = args.layers
        short = _host_capacity_shortfall(shape, psutil, whole_box=world >= torch.cuda.device_count())
        if short is not None:
            if rank == 0:
                _unavailable(f"{name} on {world} GPU(s): {short}")
            return
        mbs = micro_batch_table.get(name, 2)
        mbpr = args.micro_batches_per_rank or 1
        seq = shape["seq_len"]
        alpha = _feasible_alpha(shape, world, mbs, mbpr, getattr(args, "alpha", 0.25))
        cfg = {"max_dram_usage": psutil.virtual_memory().available / 2 ** 30,
               "batch_size": mbs * mbpr * world, "micro_batch_size": mbs, "checkpoint_interval": 1,
               # checkpoints stay in host DRAM (the reference's default): its alpha split
               # borrows that buffer for the deferred gradients and refuses alpha > 0 without it
               "split_ratio": {"checkpoint": [0.0, 1.0], "gradient": [1.0, 0.0],
                               "parameter": [0.0, 1.0], "optimizer": [0.0, 1.0], "alpha": alpha},
               "mixed_precision": {"device_dtype": "fp16", "gradacc_dtype": "fp32",
                                   "master_dtype": "fp32"}}
        init_flextrain_config(cfg)
        torch.manual_seed(0)
        t0 = time.time()
        with flextrain.Init(layer_class=Block, num_layers=shape["num_layers"],
                            param_grouping_func=lambda n, p: 1 if p.dim() == 1 else 0):
            model = Llama(shape, torch.float16, layer_device=dev, device=dev)
        decay = [p for p in model.parameters() if p.dim() > 1]
        no_decay = [p for p in model.parameters() if p.dim() <= 1]
        opt = FlexTrainAdam([{"params": decay, "weight_decay": 0.1},
                             {"params": no_decay, "weight_decay": 0.0}], lr=1e-4, betas=(0.9, 0.95))

        gen = torch.Generator().manual_seed(1 + rank)
        pool = [torch.randint(0, shape["vocab"], (mbs, seq + 1), generator=gen).pin_memory()
                for _ in range(max(64, mbpr))]
        dev_pool = [t.to(dev) for t in pool]
        state = {"i": 0, "host": False, "h2d": 0}

        def get_batch():
            i = state["i"] % len(pool)
            state["i"] += 1
            if state["host"]:
                t = pool[i].to(dev, non_blocking=True)
                state["h2d"] += pool[i].numel() * pool[i].element_size()
            else:
                t = dev_pool[i]
            return (t[:, :-1],), (), (t[:, 1:],)

        def pre_process(pre_inputs):
            (tokens,) = pre_inputs
            x = torch.nn.functional.embedding(tokens, model.embed)
            cos, sin = model.rope(tokens.shape[1], tokens.device, x.dtype)
            return (x,), (cos, sin)

        def layer_forward(start, end):
            def run(x, cos, sin):
                for i in range(start, min(end, len(model.blocks))):
                    x = model.blocks[i](x, cos, sin)
                return (x,)
            return run

        def post_process(passed_down, post_inputs):
            from baseline.llama_torch import rms_norm
            (x,) = passed_down
            return (rms_norm(x, model.final_norm),)

        def loss_fn(outputs, loss_inputs):
            (hidden,) = outputs
            (labels,) = loss_inputs
            logits = torch.nn.functional.linear(hidden, model.lm_head)
            return torch.nn.functional.cross_entropy(logits.float().view(-1, logits.shape[-1]),
                                                     labels.reshape(-1))

        flextrain.set_llm_func(lambda i: model.blocks[i], get_batch, pre_process, layer_forward,
                               post_process, loss_fn)
        engine = flextrain.initialize(model, opt)
        torch.cuda.synchronize()
        init_s = time.time() - t0

        def barrier():
            if world > 1:
                torch.distributed.barrier()
            torch.cuda.synchronize()

        def timed(steps, read_loss):
            barrier()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            last, d2h = None, 0
            for _ in range(steps):
                out = engine.train_iteration()
                if read_loss:
                    last = [float(l.detach().float().item()) for l in out]
                    d2h += 4 * len(out)
            torch.cuda.synchronize()
            e.record()
            barrier()
            ms = s.elapsed_time(e)
            if world > 1:
                t = torch.tensor([ms], device=dev)
                torch.distributed.all_reduce(t, torch.distributed.ReduceOp.MAX)
                ms = t.item()
            return ms / steps, d2h / max(steps, 1), last

        for _ in range(args.warmup):
            engine.train_iteration()
        torch.cuda.synchronize()
        ms_dev, _, _ = timed(args.steps, False)
        e2e = None
        if not args.no_e2e:
            # as many steps as the device-timed pass when the command's time limit allows it
            room = getattr(args, "wall_limit", 780.0) - (time.time() - T_START) - 20.0
            n_e2e = max(3, min(args.steps, int(room / (ms_dev / 1e3 * 1.05)) if room > 0 else 0))
            if world > 1:
                t = torch.tensor([n_e2e], device=dev)
                torch.distributed.all_reduce(t, torch.distributed.ReduceOp.MIN)
                n_e2e = int(t.item())
            state["host"], state["h2d"] = True, 0
            ms_e2e, d2h, last = timed(n_e2e, True)
            tokens = mbs * mbpr * world * seq
            e2e = {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                   "steps": n_e2e, "h2d_bytes_per_step": state["h2d"] // n_e2e,
                   "d2h_bytes_per_step": int(d2h), "last_loss": last}
        tokens = mbs * mbpr * world * seq
        if rank == 0:
            print(json.dumps({
                "metric": metric, "value": tokens / (ms_dev / 1e3), "unit": "tokens/s",
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_dev,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp16",
                "data": "synthetic", "impl": "reference",
                "config": {"model": name + (f"-{args.layers}L-DEBUG" if args.layers else ""),
                           "global_batch": mbs * mbpr * world, "micro_batch": mbs,
                           "micro_batches_per_rank": mbpr, "seq_len": seq,
                           "parallelism": f"zero3-dp{world}", "split_ratio": cfg["split_ratio"],
                           "note": "fp16 because the reference's fused Adam mis-encodes bf16; "
                                   "parameters and optimizer state in host DRAM because the "
                                   "reference asserts their GPU share to 0"},
                "e2e": e2e, "gpu_launches": 0, "init_seconds": init_s}), flush=True)
    except Exception as exc:                                   # OOM, assert inside the reference, ...
        import traceback
        traceback.print_exc(file=sys.stderr)
        if rank == 0:
            _unavailable(f"reference run failed: {type(exc).__name__}: {str(exc)[:300]}")


def _numel(s):
    kv = s["num_kv_heads"] * (s["hidden"] // s["num_heads"])
    layer = 2 * s["hidden"] + s["hidden"] * (s["hidden"] + 2 * kv) + s["hidden"] ** 2 \
        + 3 * s["hidden"] * s["ffn"]
    return layer, s["num_layers"] * layer + 2 * s["vocab"] * s["hidden"] + s["hidden"]


def _feasible_alpha(shape, world, mbs, mbpr, wanted):
    """The reference borrows its host checkpoint buffer for the gradients whose update it
    defers into the next forward pass and refuses an ``alpha`` for which those do not fit
    (``flextrain/memory/coordinator/optimizer.py:385-404``: alpha * parameters per rank and
    micro-batch must fit the checkpoint buffer of one micro-batch, in units of the fp32
    accumulation type).  Returns ``wanted`` where that holds and the largest safe value below
    it otherwise."""
    layer, _ = _numel(shape)
    ckpt = mbs * shape["seq_len"] * shape["hidden"]
    para = layer / (world * mbpr)
    bound = 0.95 * ckpt / (2.0 * para)
    return round(min(wanted, bound), 4)


def _auto_model(gpus_in_node, torch, psutil, shapes, micro_batch_table=None, args=None, policy=None):
    """The model the other arm trains on this node: the largest of the three shapes for
    which that arm's capacity planner finds a tier split on ONE GPU with its share of the
    node's host memory (the same model at every N).  The planner is a stand-alone
    pure-Python file; it is loaded by path so that nothing else of that package enters
    this process."""
    import importlib.util
    import types
    policy = policy or {"dram_share_use": 0.85, "dram_per_rank_cap": 96 * 2 ** 30}
    path = os.path.join(os.path.dirname(HERE), "flextrain_b200", "planner.py")
    spec = importlib.util.spec_from_file_location("_ft_capacity_planner", path)
    planner = importlib.util.module_from_spec(spec)
    sys.modules[spec.name] = planner          # dataclasses looks the module up by name
    spec.loader.exec_module(planner)
    hbm, _ = torch.cuda.mem_get_info()
    dram = psutil.virtual_memory().available
    share = min(dram / max(gpus_in_node, 1) * policy["dram_share_use"], policy["dram_per_rank_cap"])
    table = micro_batch_table or {}
    mbpr = (getattr(args, "micro_batches_per_rank", 0) or 1) if args is not None else 1
    buffers = getattr(args, "unit_buffers", 3) if args is not None else 3
    alpha = getattr(args, "alpha", 0.25) if args is not None else 0.25
    for name in ("llama3-70b", "llama2-13b", "llama2-7b"):
        s = dict(shapes[name])
        if args is not None and getattr(args, "seq_len", 0):
            s["seq_len"] = args.seq_len
        if args is not None and getattr(args, "layers", 0):
            s["num_layers"] = args.layers
        layer, total = _numel(s)
        cfg = types.SimpleNamespace(num_layers=s["num_layers"], layer_numel=layer, total_numel=total,
                                    hidden=s["hidden"], ffn=s["ffn"], vocab=s["vocab"], seq_len=s["seq_len"],
                                    num_heads=s["num_heads"], num_kv_heads=s["num_kv_heads"],
                                    head_dim=s["hidden"] // s["num_heads"])
        shape = planner.shape_of(cfg, table.get(name, 2))
        budget = planner.MemoryBudget(hbm, share, 0.0)
        if planner.plan(shape, 1, mbpr, budget, unit_buffers=buffers, alpha=alpha) is not None:
            return name
    return "llama2-7b"


def _host_capacity_shortfall(shape, psutil, whole_box=True):
    """The reference keeps every parameter (2 B), its fp32 master copy and both Adam
    moments (12 B) in pinned host DRAM, whatever the number of GPUs.  Returns a one-line
    reason when that exceeds what the run may take of the box's available memory - 92 %
    when the run has every GPU of the box, 60 % when others share it - else None: building
    the model anyway would pin (or exhaust) nearly all memory of a shared machine and fail
    minutes later."""
    _, total = _numel(shape)
    need = total * 14
    have = psutil.virtual_memory().available
    if need > 0.92 * have:
        whole_box = True
    if need > (0.92 if whole_box else 0.60) * have:
        return (f"the reference keeps all parameters and optimizer state in host DRAM "
                f"({need / 1e9:.0f} GB for this model) and the box offers {have / 1e9:.0f} GB"
                + ("" if whole_box else ", shared with the other GPUs' users"))
    return None
