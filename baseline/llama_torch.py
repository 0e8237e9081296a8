"""Llama-style decoder in plain PyTorch for the reference arm.

The reference ships no model, so its arm needs one; this file uses only stock
PyTorch ops (``F.linear`` -> cuBLAS, ``F.scaled_dot_product_attention``,
``F.cross_entropy``) and none of this repository's kernels, models or engine.
Same architecture and parameter shapes as the benchmark configs name: RMSNorm,
rotate-half RoPE, grouped-query causal attention, SwiGLU, untied embedding and
head, no biases.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

SHAPES = {
    "llama2-7b": dict(num_layers=32, hidden=4096, num_heads=32, num_kv_heads=32, ffn=11008,
                      vocab=32000, seq_len=4096, rope_theta=10000.0),
    "llama2-13b": dict(num_layers=40, hidden=5120, num_heads=40, num_kv_heads=40, ffn=13824,
                       vocab=32000, seq_len=4096, rope_theta=10000.0),
    "llama3-70b": dict(num_layers=80, hidden=8192, num_heads=64, num_kv_heads=8, ffn=28672,
                       vocab=128256, seq_len=4096, rope_theta=500000.0),
    "tiny": dict(num_layers=4, hidden=256, num_heads=4, num_kv_heads=4, ffn=688, vocab=1024,
                 seq_len=128, rope_theta=10000.0),
}


def rms_norm(x, w, eps=1e-5):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


def apply_rope(x, cos, sin):
    d2 = x.shape[-1] // 2
    x1, x2 = x[..., :d2], x[..., d2:]
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)


class Block(nn.Module):
    def __init__(self, shape, dtype, device=None):
        super().__init__()
        h, nh, nkv, f = shape["hidden"], shape["num_heads"], shape["num_kv_heads"], shape["ffn"]
        d = h // nh
        self.nh, self.nkv, self.d = nh, nkv, d
        mk = lambda *s: nn.Parameter(torch.empty(*s, dtype=dtype, device=device).normal_(0, 0.02))
        self.attn_norm = nn.Parameter(torch.ones(h, dtype=dtype, device=device))
        self.wqkv = mk((nh + 2 * nkv) * d, h)
        self.wo = mk(h, h)
        self.ffn_norm = nn.Parameter(torch.ones(h, dtype=dtype, device=device))
        self.w_gate_up = mk(2 * f, h)
        self.w_down = mk(h, f)

    def forward(self, x, cos, sin):
        B, S, H = x.shape
        nh, nkv, d = self.nh, self.nkv, self.d
        qkv = F.linear(rms_norm(x, self.attn_norm), self.wqkv)
        q = qkv[..., : nh * d].view(B, S, nh, d)
        k = qkv[..., nh * d:(nh + nkv) * d].view(B, S, nkv, d)
        v = qkv[..., (nh + nkv) * d:].view(B, S, nkv, d)
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                           is_causal=True, enable_gqa=nkv != nh)
        x = x + F.linear(a.transpose(1, 2).reshape(B, S, H), self.wo)
        gu = F.linear(rms_norm(x, self.ffn_norm), self.w_gate_up)
        g, u = gu.chunk(2, dim=-1)
        return x + F.linear(F.silu(g) * u, self.w_down)


class Llama(nn.Module):
    def __init__(self, shape, dtype, layer_device=None, device=None):
        super().__init__()
        self.shape = shape
        h, v = shape["hidden"], shape["vocab"]
        self.embed = nn.Parameter(torch.empty(v, h, dtype=dtype, device=device).normal_(0, 0.02))
        self.blocks = nn.ModuleList([Block(shape, dtype, layer_device) for _ in range(shape["num_layers"])])
        self.final_norm = nn.Parameter(torch.ones(h, dtype=dtype, device=device))
        self.lm_head = nn.Parameter(torch.empty(v, h, dtype=dtype, device=device).normal_(0, 0.02))

    def rope(self, seq, device, dtype):
        d = self.shape["hidden"] // self.shape["num_heads"]
        inv = 1.0 / (self.shape["rope_theta"] ** (torch.arange(0, d, 2, device=device).float() / d))
        fr = torch.outer(torch.arange(seq, device=device).float(), inv)
        return fr.cos().to(dtype), fr.sin().to(dtype)
