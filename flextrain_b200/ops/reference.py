"""Plain PyTorch statements of every model op.

They are the CPU backend of ``ops.functional`` (gloo runs, tests without a GPU)
and the oracle the sm_100a kernels are checked against.  All math is done in
fp32 and cast back to the input dtype.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x @ w.T`` with ``w`` stored ``[out_features, in_features]``."""
    return F.linear(x, w)


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    inv = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (xf * inv * weight.float()).to(x.dtype)


def layernorm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    mean = xf.mean(-1, keepdim=True)
    var = (xf - mean).pow(2).mean(-1, keepdim=True)
    return ((xf - mean) * torch.rsqrt(var + eps) * weight.float() + bias.float()).to(x.dtype)


def bias_add(x: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    return (x.float() + bias.float()).to(x.dtype)


def bias_gelu(x: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """tanh-approximated GELU of ``x + bias`` (the GPT-2 / Megatron form)."""
    return F.gelu(x.float() + bias.float(), approximate="tanh").to(x.dtype)


def rope_tables(seq_len: int, head_dim: int, theta: float, device=None,
                dtype=torch.float32) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos/sin tables of shape ``[seq_len, head_dim // 2]``."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32)
                                / head_dim))
    t = torch.arange(seq_len, device=device, dtype=torch.float32)
    freqs = torch.outer(t, inv_freq)
    return freqs.cos().to(dtype), freqs.sin().to(dtype)


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half RoPE.  ``x``: ``[B, S, H, D]``; ``cos``/``sin``: ``[S, D/2]``.
    Pairs are ``(x[..., i], x[..., i + D/2])``."""
    d2 = x.shape[-1] // 2
    xf = x.float()
    x1, x2 = xf[..., :d2], xf[..., d2:]
    c = cos.float()[None, :, None, :]
    s = sin.float()[None, :, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` for ``gate_up = [gate | up]`` along the last dim."""
    f = gate_up.shape[-1] // 2
    g, u = gate_up[..., :f].float(), gate_up[..., f:].float()
    return (F.silu(g) * u).to(gate_up.dtype)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                     scale: Optional[float] = None) -> torch.Tensor:
    """Causal softmax attention.  ``q``: ``[B, S, H, D]``; ``k``/``v``:
    ``[B, S, Hkv, D]`` with ``H % Hkv == 0`` (grouped-query attention)."""
    B, S, H, D = q.shape
    hkv = k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(H // hkv, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(H // hkv, dim=1)
    scores = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    mask = torch.ones(S, S, dtype=torch.bool, device=q.device).tril_()
    scores = scores.masked_fill(~mask, float("-inf"))
    out = torch.matmul(torch.softmax(scores, dim=-1), vf)
    return out.permute(0, 2, 1, 3).to(q.dtype)


def cross_entropy(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100):
    """Mean token cross-entropy over ``[N, V]`` logits."""
    return F.cross_entropy(logits.float(), labels, ignore_index=ignore_index)


def linear_cross_entropy(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor,
                         ignore_index: int = -100) -> torch.Tensor:
    """``cross_entropy(hidden @ weight.T, labels)`` (mean over valid tokens)."""
    return cross_entropy(F.linear(hidden, weight), labels, ignore_index)
