#!/usr/bin/env python
"""Bring your own model: a stack of stock ``torch.nn`` blocks trained through the engine.

    python examples/custom_model.py [--steps 20] [--device cpu|cuda] [--offload]

The six callbacks below are everything the engine needs to know about a model
(the contract of flextrain/llm_func.py:8-33):

    get_batch()                      -> (pre_inputs, post_inputs, loss_inputs) of one micro-batch
    pre_process(pre_inputs)          -> (passed_down, every_layer): one tensor that flows from
                                        layer to layer, plus constants every layer receives
    layer_forward(start, end)        -> callable running layers [start, end) on passed_down
    post_process(passed_down, post)  -> model outputs
    loss(outputs, loss_inputs)       -> the loss (or a tuple whose first one-element tensor is it)
    get_layer(i)                     -> layer i (kept for scripts that use it; the engine does not)

``flextrain.Init`` watches the constructor of the layer class: the parameters of every
``checkpoint_interval`` consecutive layers become one unit that is partitioned over the
ranks and placed on HBM / host memory / NVMe by ``split_ratio``.  With ``--offload`` half of
the parameters and all optimizer state live in host memory; the losses are the same.
"""
import argparse
import os
import sys

import torch
import torch.nn as nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import flextrain_b200 as flextrain  # noqa: E402
from flextrain_b200.config import init_flextrain_config  # noqa: E402
from flextrain_b200.ops.adam import FlexTrainAdam  # noqa: E402


class Block(nn.Module):
    def __init__(self, width):
        super().__init__()
        self.norm = nn.LayerNorm(width)
        self.fc1 = nn.Linear(width, 4 * width)
        self.fc2 = nn.Linear(4 * width, width)

    def forward(self, x):
        return x + self.fc2(torch.nn.functional.gelu(self.fc1(self.norm(x))))


class Regressor(nn.Module):
    def __init__(self, features, width, depth):
        super().__init__()
        self.inp = nn.Linear(features, width)
        self.blocks = nn.ModuleList([Block(width) for _ in range(depth)])
        self.out = nn.Linear(width, 1)


def main():
    ap = argparse.ArgumentParser()
    flextrain.add_config_arguments(ap)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--offload", action="store_true")
    ap.add_argument("--depth", type=int, default=6)
    ap.add_argument("--width", type=int, default=64)
    args = ap.parse_args()

    on_gpu = args.device == "cuda"
    flextrain.init_distributed(dist_backend="nccl" if on_gpu else "gloo", force_init=False)
    rank, world = flextrain.distributed.get_rank(), flextrain.distributed.get_world_size()
    device = flextrain.distributed.current_device()
    micro_batch, micro_batches_per_rank = 8, 2
    first = [0.5, 0.5] if args.offload else [1.0, 0.0]
    init_flextrain_config({
        "batch_size": micro_batch * micro_batches_per_rank * world, "micro_batch_size": micro_batch,
        "checkpoint_interval": 2,
        "mixed_precision": {"device_dtype": "fp32"},
        "split_ratio": {"parameter": first, "optimizer": [0.0, 1.0] if args.offload else [1.0, 0.0],
                        "checkpoint": first, "gradient": [1.0, 0.0], "alpha": 0.25},
    })

    torch.manual_seed(0)
    with flextrain.Init(layer_class=Block, num_layers=args.depth):
        model = Regressor(16, args.width, args.depth).to(device)
    decay = [p for n, p in model.named_parameters() if p.dim() > 1]
    rest = [p for n, p in model.named_parameters() if p.dim() <= 1]
    optimizer = FlexTrainAdam([{"params": decay, "weight_decay": 0.01}, {"params": rest, "weight_decay": 0.0}],
                              lr=3e-3)

    # a fixed synthetic regression task: y = sin of a random projection of x
    gen = torch.Generator().manual_seed(1 + rank)
    proj = torch.randn(16, 1, generator=torch.Generator().manual_seed(7)) / 4

    def get_batch():
        x = torch.randn(micro_batch, 16, generator=gen)
        y = torch.sin(x @ proj)
        return (x.to(device),), (), (y.to(device),)

    def pre_process(pre_inputs):
        return (model.inp(pre_inputs[0]),), ()

    def layer_forward(start, end):
        def run(h):
            for i in range(start, min(end, len(model.blocks))):
                h = model.blocks[i](h)
            return (h,)
        return run

    def post_process(passed_down, post_inputs):
        return (model.out(passed_down[0]),)

    def loss_fn(outputs, loss_inputs):
        return ((outputs[0] - loss_inputs[0]) ** 2).mean()

    flextrain.set_llm_func(lambda i: model.blocks[i], get_batch, pre_process, layer_forward, post_process,
                           loss_fn)
    engine = flextrain.initialize(model, optimizer)
    losses = []
    for step in range(args.steps):
        results = engine.train_iteration()                 # one entry per local micro-batch
        local = sum(float(r.detach()) for r in results) / len(results)
        losses.append(flextrain.distributed.all_reduce_scalar(local) / world)
        if (step + 1) % 5 == 0:
            flextrain.distributed.print_rank0(f"step {step + 1:4d}  loss {losses[-1]:.5f}")
    engine.shutdown()
    if rank == 0:
        print(f"first loss {losses[0]:.5f}  last loss {losses[-1]:.5f}", flush=True)


if __name__ == "__main__":
    main()
