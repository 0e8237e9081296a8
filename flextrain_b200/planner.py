"""Closed-form tier planner: choose split ratios for a Llama-shape model from
memory capacities alone (no profiling run).

The profiling planner of ``auto_config`` measures the machine and solves an LP;
this module is its zero-cost sibling used by ``bench.py`` and as the starting
point of ``auto_config``.  Unlike the reference's planner
(flextrain/auto_config.py:404-422, no GPU variables for parameters, optimizer
state or checkpoints) HBM is the first tier: what does not fit there goes to
host DRAM, then to NVMe.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

GiB = float(1 << 30)


@dataclass
class MemoryBudget:
    hbm_bytes: float          # usable HBM per GPU
    dram_bytes: float         # usable host DRAM per rank
    nvme_bytes: float = 0.0   # usable NVMe per rank


@dataclass
class ModelShape:
    num_layers: int
    layer_numel: int
    nonlayer_numel: int
    hidden: int
    ffn: int
    vocab: int
    tokens_per_micro_batch: int
    kv_dim: int

    @property
    def total_numel(self) -> int:
        return self.num_layers * self.layer_numel + self.nonlayer_numel


def shape_of(cfg, micro_batch_size: int) -> ModelShape:
    """Shape of a model config of ``models.llama`` or ``models.gpt`` (anything with
    ``num_layers``, ``layer_numel``, ``total_numel``, ``hidden``, ``ffn``, ``vocab``,
    ``seq_len``, ``num_heads`` and optionally ``num_kv_heads``)."""
    kv_heads = getattr(cfg, "num_kv_heads", None) or cfg.num_heads
    return ModelShape(cfg.num_layers, cfg.layer_numel, cfg.total_numel - cfg.num_layers * cfg.layer_numel,
                      cfg.hidden, cfg.ffn, cfg.vocab, micro_batch_size * cfg.seq_len,
                      kv_heads * cfg.head_dim)


def activation_bytes(s: ModelShape, interval: int = 1) -> float:
    """Peak bytes of one unit's autograd graph for one micro-batch (bf16)."""
    per_token = (4 * s.hidden + 2 * (s.hidden + 2 * s.kv_dim) + 2 * s.hidden   # norms, qkv(+roped), attn
                 + 3 * 2 * s.ffn + s.ffn + 2 * s.hidden) * 2.0
    head = min(4096, s.tokens_per_micro_batch) * s.vocab * 2.0 * 2
    return per_token * s.tokens_per_micro_batch * interval * 1.25 + head


def working_set_bytes(s: ModelShape, world: int, mbpr: int, unit_buffers: int = 3,
                      wide_accumulate: bool = True, interval: int = 1) -> float:
    unit = s.layer_numel * interval
    ws = unit_buffers * unit * 2.0                     # gathered unit ring
    ws += 2 * unit * (2.0 + (4.0 if wide_accumulate and mbpr > 1 else 0.0))   # gradient buffers
    ws += s.nonlayer_numel * (2.0 + 2.0 + 12.0)        # replicated params, grads, fp32 state
    ws += activation_bytes(s, interval)
    ws += 2 * s.tokens_per_micro_batch * s.hidden * 2.0 * 2   # activation gradient + slack
    return ws


def plan(s: ModelShape, world: int, mbpr: int, budget: MemoryBudget, unit_buffers: int = 3,
         interval: int = 1, alpha: float = 0.25, headroom: float = 0.06) -> Optional[Dict]:
    """Split ratios for ``config['split_ratio']`` or None when the model's state
    cannot be held by HBM + DRAM + NVMe of ``world`` ranks."""
    units = -(-s.num_layers // interval)
    unit = s.layer_numel * interval
    shard_params = units * unit / world
    para_bytes = shard_params * 2.0
    opts_bytes = shard_params * 12.0
    ckpt_bytes = units * mbpr * s.tokens_per_micro_batch * s.hidden * 2.0
    hbm = budget.hbm_bytes * (1.0 - headroom) - working_set_bytes(s, world, mbpr, unit_buffers,
                                                                 True, interval)
    dram = budget.dram_bytes
    nvme = budget.nvme_bytes
    if hbm <= 0:
        return None

    def place(need, hbm_left, dram_left, nvme_left, pinned_cost=1.0):
        g = min(need, max(hbm_left, 0.0))
        c = min(need - g, max(dram_left, 0.0) / pinned_cost)
        n = need - g - c
        return g, c, n

    # order: parameters (read twice per step), checkpoints, optimizer state
    pg, pc, pn = place(para_bytes, hbm, dram, nvme)
    hbm, dram, nvme = hbm - pg, dram - pc, nvme - pn
    kg, kc, kn = place(ckpt_bytes, hbm, dram, nvme)
    hbm, dram, nvme = hbm - kg, dram - kc, nvme - kn
    # host gradients + staging for the DRAM share of the optimizer: ~ (4+2)/12 of two units
    og, oc, on = place(opts_bytes, hbm, dram * 0.92, nvme)
    hbm, dram, nvme = hbm - og, dram - oc, nvme - on
    if nvme < -1.0:
        return None

    def ratio(g, c, total):
        if total <= 0:
            return [1.0, 0.0]
        gr, cr = g / total, c / total
        # keep a hair below the exact share so page rounding never overshoots the budget
        return [max(0.0, round(gr - 5e-4, 4)) if 0 < gr < 1 else round(gr, 4),
                round(min(1.0 - max(0.0, gr), cr + (5e-4 if 0 < gr < 1 and pn + kn + on == 0 else 0)), 4)]

    out = {"parameter": ratio(pg, pc, para_bytes), "checkpoint": ratio(kg, kc, ckpt_bytes),
           "optimizer": ratio(og, oc, opts_bytes), "gradient": [1.0, 0.0], "alpha": alpha}
    for k in ("parameter", "checkpoint", "optimizer"):
        g_, c_ = out[k]
        if g_ + c_ > 1.0:
            out[k] = [g_, round(1.0 - g_, 4)]
        if (k == "parameter" and pn == 0) or (k == "checkpoint" and kn == 0) or \
                (k == "optimizer" and on == 0):
            out[k] = [out[k][0], round(1.0 - out[k][0], 4)]
    return out


def fits(s: ModelShape, world: int, mbpr: int, budget: MemoryBudget, **kw) -> bool:
    return plan(s, world, mbpr, budget, **kw) is not None
