"""GPT-2 / Megatron-GPT style decoder built on the package's ops and exposed
through the pre / layer / post callback split the engine drives.

The reference ships no model: its users bring Megatron-LM's GPT, whose blocks
are pre-LayerNorm, biased projections, multi-head causal attention, a 4x MLP
with the tanh GELU fused with its bias, learned absolute position embeddings and
a head tied to the token embedding (the reference's checkpointing module keeps
Megatron's RNG-tracker interface for exactly that user, flextrain/checkpointing.py:63-189).
This module supplies that architecture so the second model family of the
reference's users runs on the same engine as ``models.llama``.  QKV is stored
fused (``[q heads | k heads | v heads]`` along the output dimension) so the
projection is one GEMM and the packed attention kernels read it in place.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional, Tuple

import torch
import torch.nn as nn

from ..ops import functional as F


@dataclass
class GPTConfig:
    num_layers: int = 4
    hidden: int = 256
    num_heads: int = 4
    ffn: Optional[int] = None            # 4 * hidden when not given
    vocab: int = 1024
    seq_len: int = 128                   # rows of the position table
    eps: float = 1e-5
    init_std: float = 0.02
    tie_embeddings: bool = True
    dropout: float = 0.0                 # embedding and residual-branch dropout (GPT-2: 0.1)
    name: str = "tiny"

    def __post_init__(self):
        if self.ffn is None:
            self.ffn = 4 * self.hidden
        if self.hidden % self.num_heads:
            raise ValueError("hidden must divide by heads")
        if not 0.0 <= self.dropout < 1.0:
            raise ValueError("dropout must lie in [0, 1)")

    @property
    def head_dim(self) -> int:
        return self.hidden // self.num_heads

    @property
    def layer_numel(self) -> int:
        h, f = self.hidden, self.ffn
        return 4 * h + (3 * h * h + 3 * h) + (h * h + h) + (f * h + f) + (h * f + h)

    @property
    def total_numel(self) -> int:
        head = 0 if self.tie_embeddings else self.vocab * self.hidden
        return self.num_layers * self.layer_numel + self.vocab * self.hidden \
            + self.seq_len * self.hidden + 2 * self.hidden + head


PRESETS = {
    "tiny": dict(num_layers=4, hidden=256, num_heads=4, vocab=1024, seq_len=128),
    "gpt2-small": dict(num_layers=12, hidden=768, num_heads=12, vocab=50304, seq_len=1024),
    "gpt2-medium": dict(num_layers=24, hidden=1024, num_heads=16, vocab=50304, seq_len=1024),
    "gpt2-large": dict(num_layers=36, hidden=1280, num_heads=20, vocab=50304, seq_len=1024),
    "gpt2-xl": dict(num_layers=48, hidden=1600, num_heads=25, vocab=50304, seq_len=1024),
    "gpt3-6.7b": dict(num_layers=32, hidden=4096, num_heads=32, vocab=50304, seq_len=2048),
    "gpt3-13b": dict(num_layers=40, hidden=5120, num_heads=40, vocab=50304, seq_len=2048),
    "gpt3-175b": dict(num_layers=96, hidden=12288, num_heads=96, vocab=50304, seq_len=2048),
}


def preset(name: str, **overrides) -> GPTConfig:
    cfg = dict(PRESETS[name])
    cfg.update(overrides)
    return GPTConfig(name=name, **cfg)


class GPTBlock(nn.Module):
    # the parameter the block multiplies first: on several GPUs the engine may leave it out of
    # the layer's parameter gather and let that product fetch it (all-gather fused into the GEMM)
    ft_first_gemm_weight = "wqkv"

    def __init__(self, cfg: GPTConfig, dtype=torch.float32, layer_index: int = 0):
        super().__init__()
        self.cfg = cfg
        h, f = cfg.hidden, cfg.ffn
        mk = lambda *shape: nn.Parameter(torch.empty(*shape, dtype=dtype))      # noqa: E731
        self.ln1_w, self.ln1_b = nn.Parameter(torch.ones(h, dtype=dtype)), nn.Parameter(torch.zeros(h, dtype=dtype))
        self.wqkv, self.bqkv = mk(3 * h, h), nn.Parameter(torch.zeros(3 * h, dtype=dtype))
        self.wo, self.bo = mk(h, h), nn.Parameter(torch.zeros(h, dtype=dtype))
        self.ln2_w, self.ln2_b = nn.Parameter(torch.ones(h, dtype=dtype)), nn.Parameter(torch.zeros(h, dtype=dtype))
        self.w_fc, self.b_fc = mk(f, h), nn.Parameter(torch.zeros(f, dtype=dtype))
        self.w_proj, self.b_proj = mk(h, f), nn.Parameter(torch.zeros(h, dtype=dtype))
        for w in (self.wqkv, self.w_fc):
            nn.init.normal_(w, mean=0.0, std=cfg.init_std)
        # residual-path projections: std / sqrt(2 * layers), as GPT-2 and Megatron do
        for w in (self.wo, self.w_proj):
            nn.init.normal_(w, mean=0.0, std=cfg.init_std / (2.0 * cfg.num_layers) ** 0.5)

    def _drop(self, t: torch.Tensor) -> torch.Tensor:
        # masks come from the default generator: the engine's checkpointing saves and
        # replays its state, so the recomputed forward draws the same masks
        p = self.cfg.dropout
        return torch.nn.functional.dropout(t, p, True) if p > 0.0 and self.training else t

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        B, S, H = x.shape
        nh, d = cfg.num_heads, cfg.head_dim
        h = F.layernorm(x, self.ln1_w, self.ln1_b, cfg.eps)
        qkv = F.bias_add(F.linear(h, self.wqkv), self.bqkv)
        a = F.attention_packed(qkv, nh, nh, d) if qkv.is_cuda else None
        if a is None:
            q, k, v = (t.unflatten(-1, (nh, d)) for t in qkv.split(H, dim=-1))
            a = F.causal_attention(q, k, v).reshape(B, S, H)
        x = x + self._drop(F.bias_add(F.linear(a, self.wo), self.bo))
        h = F.layernorm(x, self.ln2_w, self.ln2_b, cfg.eps)
        h = F.bias_gelu(F.linear(h, self.w_fc), self.b_fc)
        return x + self._drop(F.bias_add(F.linear(h, self.w_proj), self.b_proj))


class GPTModel(nn.Module):
    """Token + position embedding, ``num_layers`` blocks, final LayerNorm and
    head (tied to the token embedding unless ``tie_embeddings`` is off).  Build
    it inside ``flextrain.Init(layer_class=GPTBlock, ...)`` to have the blocks
    partitioned as they are created."""

    def __init__(self, cfg: GPTConfig, dtype=torch.float32, device=None):
        super().__init__()
        self.cfg = cfg
        self.wte = nn.Parameter(torch.empty(cfg.vocab, cfg.hidden, dtype=dtype, device=device))
        self.wpe = nn.Parameter(torch.empty(cfg.seq_len, cfg.hidden, dtype=dtype, device=device))
        nn.init.normal_(self.wte, mean=0.0, std=cfg.init_std)
        nn.init.normal_(self.wpe, mean=0.0, std=cfg.init_std)
        self.blocks = nn.ModuleList([GPTBlock(cfg, dtype=dtype, layer_index=i)
                                     for i in range(cfg.num_layers)])
        self.lnf_w = nn.Parameter(torch.ones(cfg.hidden, dtype=dtype, device=device))
        self.lnf_b = nn.Parameter(torch.zeros(cfg.hidden, dtype=dtype, device=device))
        if cfg.tie_embeddings:
            self.lm_head = None
        else:
            self.lm_head = nn.Parameter(torch.empty(cfg.vocab, cfg.hidden, dtype=dtype, device=device))
            nn.init.normal_(self.lm_head, mean=0.0, std=cfg.init_std)

    # the three stages, also usable without the engine
    def pre_process(self, tokens: torch.Tensor) -> torch.Tensor:
        S = tokens.shape[1]
        if S > self.cfg.seq_len:
            raise ValueError(f"sequence of {S} tokens exceeds the position table ({self.cfg.seq_len})")
        x = torch.nn.functional.embedding(tokens, self.wte) + self.wpe[:S]
        p = self.cfg.dropout
        return torch.nn.functional.dropout(x, p, True) if p > 0.0 and self.training else x

    def post_process(self, x: torch.Tensor) -> torch.Tensor:
        return F.layernorm(x, self.lnf_w, self.lnf_b, self.cfg.eps)

    def loss(self, hidden: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        head = self.wte if self.lm_head is None else self.lm_head
        return F.linear_cross_entropy(hidden.reshape(-1, hidden.shape[-1]), head, labels.reshape(-1))

    def forward(self, tokens: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        x = self.pre_process(tokens)
        for blk in self.blocks:
            x = blk(x)
        return self.loss(self.post_process(x), labels)


def param_grouping(name: str, p: torch.Tensor) -> int:
    """0: weight-decayed matrices, 1: gains and biases (no decay)."""
    return 1 if p.dim() == 1 else 0


def make_param_groups(model: GPTModel, weight_decay: float = 0.0, lr: Optional[float] = None):
    decay = [p for p in model.parameters() if p.dim() > 1]
    no_decay = [p for p in model.parameters() if p.dim() <= 1]
    groups = [{"params": decay, "weight_decay": weight_decay},
              {"params": no_decay, "weight_decay": 0.0}]
    if lr is not None:
        for g in groups:
            g["lr"] = lr
    return groups


def make_llm_funcs(model: GPTModel, batch_fn: Callable[[], Tuple[torch.Tensor, torch.Tensor]]):
    """The six callbacks for ``set_llm_func``.  ``batch_fn()`` returns one
    micro-batch ``(tokens [B, S] int64, labels [B, S] int64)`` on the compute
    device."""

    def get_layer(i):
        return model.blocks[i]

    def get_batch():
        tokens, labels = batch_fn()
        return (tokens,), (), (labels,)

    def pre_process(pre_inputs):
        (tokens,) = pre_inputs
        return (model.pre_process(tokens),), ()

    def layer_forward(start, end):
        def run(x):
            for i in range(start, min(end, len(model.blocks))):
                x = model.blocks[i](x)
            return (x,)
        return run

    def post_process(passed_down, post_inputs):
        (x,) = passed_down
        return (model.post_process(x),)

    def loss(outputs, loss_inputs):
        (hidden,) = outputs
        (labels,) = loss_inputs
        return model.loss(hidden, labels)

    return get_layer, get_batch, pre_process, layer_forward, post_process, loss
