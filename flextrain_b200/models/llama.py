"""Llama-style decoder built on the package's ops and exposed through the
pre / layer / post callback split the engine drives.

The reference ships no model (its users bring a Megatron-style one); this
module supplies the architecture named by the benchmark configs: RMSNorm,
rotary embeddings (rotate-half), grouped-query causal attention, SwiGLU FFN,
untied embedding and head, no biases.  QKV and gate/up projections are stored
fused so each is one GEMM.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional, Tuple

import torch
import torch.nn as nn

from ..ops import functional as F


@dataclass
class LlamaConfig:
    num_layers: int = 4
    hidden: int = 256
    num_heads: int = 4
    num_kv_heads: Optional[int] = None
    ffn: int = 688
    vocab: int = 1024
    eps: float = 1e-5
    rope_theta: float = 10000.0
    seq_len: int = 128
    init_std: float = 0.02
    name: str = "tiny"

    def __post_init__(self):
        if self.num_kv_heads is None:
            self.num_kv_heads = self.num_heads
        if self.hidden % self.num_heads or self.num_heads % self.num_kv_heads:
            raise ValueError("hidden must divide by heads and heads by kv heads")

    @property
    def head_dim(self) -> int:
        return self.hidden // self.num_heads

    @property
    def layer_numel(self) -> int:
        kv = self.num_kv_heads * self.head_dim
        return 2 * self.hidden + self.hidden * (self.hidden + 2 * kv) + self.hidden * self.hidden \
            + 3 * self.hidden * self.ffn

    @property
    def total_numel(self) -> int:
        return self.num_layers * self.layer_numel + 2 * self.vocab * self.hidden + self.hidden


PRESETS = {
    "tiny": dict(num_layers=4, hidden=256, num_heads=4, ffn=688, vocab=1024, seq_len=128,
                 rope_theta=10000.0),
    "llama2-7b": dict(num_layers=32, hidden=4096, num_heads=32, ffn=11008, vocab=32000,
                      seq_len=4096, rope_theta=10000.0),
    "llama2-13b": dict(num_layers=40, hidden=5120, num_heads=40, ffn=13824, vocab=32000,
                       seq_len=4096, rope_theta=10000.0),
    "llama3-70b": dict(num_layers=80, hidden=8192, num_heads=64, num_kv_heads=8, ffn=28672,
                       vocab=128256, seq_len=4096, rope_theta=500000.0),
}


def preset(name: str, **overrides) -> LlamaConfig:
    cfg = dict(PRESETS[name])
    cfg.update(overrides)
    return LlamaConfig(name=name, **cfg)


class LlamaBlock(nn.Module):
    # the parameter the block multiplies first: on several GPUs the engine may leave it out of
    # the layer's parameter gather and let that product fetch it (all-gather fused into the GEMM)
    ft_first_gemm_weight = "wqkv"

    def __init__(self, cfg: LlamaConfig, dtype=torch.float32):
        super().__init__()
        self.cfg = cfg
        h, d = cfg.hidden, cfg.head_dim
        kv = cfg.num_kv_heads * d
        self.attn_norm = nn.Parameter(torch.ones(h, dtype=dtype))
        self.wqkv = nn.Parameter(torch.empty(h + 2 * kv, h, dtype=dtype))
        self.wo = nn.Parameter(torch.empty(h, h, dtype=dtype))
        self.ffn_norm = nn.Parameter(torch.ones(h, dtype=dtype))
        self.w_gate_up = nn.Parameter(torch.empty(2 * cfg.ffn, h, dtype=dtype))
        self.w_down = nn.Parameter(torch.empty(h, cfg.ffn, dtype=dtype))
        for w in (self.wqkv, self.wo, self.w_gate_up, self.w_down):
            nn.init.normal_(w, mean=0.0, std=cfg.init_std)

    def forward(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        B, S, H = x.shape
        d, nh, nkv = cfg.head_dim, cfg.num_heads, cfg.num_kv_heads
        h = F.rmsnorm(x, self.attn_norm, cfg.eps)
        qkv = F.linear(h, self.wqkv)
        if qkv.is_cuda:
            # rotate the q and k heads inside the fused projection; q, k, v stay views
            qkv = F.rope_heads_inplace(qkv, cos, sin, nh + nkv, d)
            packed = F.attention_packed(qkv, nh, nkv, d)
            if packed is not None:
                x, h = F.add_rmsnorm(x, F.linear(packed, self.wo), self.ffn_norm, cfg.eps)
                return F.linear_add(F.linear_swiglu(h, self.w_gate_up), self.w_down, x)
        q = qkv[..., : nh * d].unflatten(-1, (nh, d))
        k = qkv[..., nh * d: (nh + nkv) * d].unflatten(-1, (nkv, d))
        v = qkv[..., (nh + nkv) * d:].unflatten(-1, (nkv, d))
        if not qkv.is_cuda:
            q, k = F.rope(q, cos, sin), F.rope(k, cos, sin)
        a = F.causal_attention(q, k, v).reshape(B, S, H)
        x, h = F.add_rmsnorm(x, F.linear(a, self.wo), self.ffn_norm, cfg.eps)
        return F.linear_add(F.linear_swiglu(h, self.w_gate_up), self.w_down, x)


class LlamaModel(nn.Module):
    """Embedding, ``num_layers`` blocks, final norm and head.  Build it inside
    ``flextrain.Init(layer_class=LlamaBlock, ...)`` to have the blocks
    partitioned as they are created."""

    def __init__(self, cfg: LlamaConfig, dtype=torch.float32, device=None):
        super().__init__()
        self.cfg = cfg
        self.embed = nn.Parameter(torch.empty(cfg.vocab, cfg.hidden, dtype=dtype, device=device))
        nn.init.normal_(self.embed, mean=0.0, std=cfg.init_std)
        self.blocks = nn.ModuleList([LlamaBlock(cfg, dtype=dtype) for _ in range(cfg.num_layers)])
        self.final_norm = nn.Parameter(torch.ones(cfg.hidden, dtype=dtype, device=device))
        self.lm_head = nn.Parameter(torch.empty(cfg.vocab, cfg.hidden, dtype=dtype, device=device))
        nn.init.normal_(self.lm_head, mean=0.0, std=cfg.init_std)
        self._rope_cache = {}

    def rope(self, seq_len: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
        key = (seq_len, str(device))
        if key not in self._rope_cache:
            self._rope_cache[key] = F.rope_tables(seq_len, self.cfg.head_dim, self.cfg.rope_theta,
                                                  device=device)
        return self._rope_cache[key]

    # the three stages, also usable without the engine
    def pre_process(self, tokens: torch.Tensor):
        x = torch.nn.functional.embedding(tokens, self.embed)
        cos, sin = self.rope(tokens.shape[1], tokens.device)
        return x, cos, sin

    def post_process(self, x: torch.Tensor) -> torch.Tensor:
        return F.rmsnorm(x, self.final_norm, self.cfg.eps)

    def loss(self, hidden: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        return F.linear_cross_entropy(hidden.reshape(-1, hidden.shape[-1]), self.lm_head,
                                      labels.reshape(-1))

    def forward(self, tokens: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        x, cos, sin = self.pre_process(tokens)
        for blk in self.blocks:
            x = blk(x, cos, sin)
        return self.loss(self.post_process(x), labels)


def param_grouping(name: str, p: torch.Tensor) -> int:
    """0: weight-decayed matrices, 1: norm gains (no decay)."""
    return 1 if p.dim() == 1 else 0


def make_param_groups(model: LlamaModel, weight_decay: float = 0.0, lr: Optional[float] = None):
    decay = [p for p in model.parameters() if p.dim() > 1]
    no_decay = [p for p in model.parameters() if p.dim() <= 1]
    groups = [{"params": decay, "weight_decay": weight_decay},
              {"params": no_decay, "weight_decay": 0.0}]
    if lr is not None:
        for g in groups:
            g["lr"] = lr
    return groups


def make_llm_funcs(model: LlamaModel, batch_fn: Callable[[], Tuple[torch.Tensor, torch.Tensor]]):
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
        x, cos, sin = model.pre_process(tokens)
        return (x,), (cos, sin)

    def layer_forward(start, end):
        def run(x, cos, sin):
            for i in range(start, min(end, len(model.blocks))):
                x = model.blocks[i](x, cos, sin)
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
