"""Python front of the fused compute + collective kernels.

``FusedReduceScatterAdam``: gradient reduce-scatter over peer memory fused with
unscale, finite check, the HBM share of Adam and the hand-off of the host share
(``csrc/comm/rs_adam.cu``).  It replaces, call for call, the sequence NCCL
reduce-scatter -> finite flag -> device Adam -> device-to-host gradient copy of
``memory/coordinator/optimizer.py``.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_int64, c_uint32, c_void_p
from typing import Dict, Optional, Sequence

import torch

from ..ops.native import cuda_lib, dtype_code, ptr, stream_handle
from ..param_group import GroupSegment


class _AdamSegment(ctypes.Structure):
    _fields_ = [("lo", c_int64), ("hi", c_int64), ("lr", c_float), ("beta1", c_float),
                ("beta2", c_float), ("eps", c_float), ("weight_decay", c_float), ("adamw", c_int),
                ("bias_correction", c_int), ("step", c_int64)]


_DECLARED = False


def _lib():
    global _DECLARED
    lib = cuda_lib()
    if not _DECLARED:
        lib.ft_rs_adam.argtypes = [
            c_int, c_int, c_void_p, c_void_p, c_int, c_int64, c_float, c_uint32, c_int, c_int,
            c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int,
            c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p]
        lib.ft_ar_adam.argtypes = [
            c_int, c_int, c_void_p, c_void_p, c_int, c_int64, c_float, c_uint32, c_int, c_int,
            c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p,
            c_int, c_void_p]
        lib.ft_comm_error.restype = c_int
        _DECLARED = True
    return lib


def make_segments(segments: Sequence[GroupSegment], param_groups: Sequence[Dict], defaults_owner,
                  step: int):
    d = defaults_owner.defaults
    arr = (_AdamSegment * max(len(segments), 1))()
    for i, seg in enumerate(segments):
        g = param_groups[seg.group]
        b1, b2 = g.get("betas", d["betas"])
        arr[i] = _AdamSegment(seg.start, seg.end, g.get("lr", d["lr"]), b1, b2, g.get("eps", d["eps"]),
                              g.get("weight_decay", d["weight_decay"]),
                              int(getattr(defaults_owner, "adamw_mode", True)),
                              int(g.get("bias_correction", d["bias_correction"])), int(step))
    return arr


def segments_aligned(segments: Sequence[GroupSegment], *bounds: int) -> bool:
    return all(s.start % 8 == 0 and s.end % 8 == 0 for s in segments) and \
        all(b % 8 == 0 for b in bounds) and len(segments) <= 8


def rs_adam(world: int, rank: int, grad_ptrs, flag_ptrs, grad_dtype: torch.dtype, shard: int,
            scale: float, seq: int, reduced_out: Optional[torch.Tensor], og: int, do_adam: bool,
            master: Optional[torch.Tensor], m: Optional[torch.Tensor], v: Optional[torch.Tensor],
            param_a: Optional[torch.Tensor], a_hi: int, param_b: Optional[torch.Tensor],
            param_dtype: torch.dtype, host_grad: Optional[torch.Tensor],
            finite_flag: Optional[torch.Tensor], segments, nseg: int, max_blocks: int = 148,
            start_slot: int = 0, done_slot: int = 1, status: Optional[torch.Tensor] = None):
    """Thin wrapper over ``ft_rs_adam``; see ``csrc/comm/rs_adam.cu``.  ``status`` (one int32,
    pinned host or device memory) receives 101 when this rank gave up waiting for its peers
    at the start of the call, in which case none of the outputs was written."""
    rc = _lib().ft_rs_adam(
        world, rank, ctypes.cast(grad_ptrs, c_void_p), ctypes.cast(flag_ptrs, c_void_p) if flag_ptrs
        is not None else None, dtype_code(grad_dtype), shard, float(scale), seq, start_slot, done_slot,
        ptr(reduced_out), og, int(do_adam), ptr(master), ptr(m), ptr(v), ptr(param_a), a_hi,
        ptr(param_b), dtype_code(param_dtype), ptr(host_grad),
        -1 if host_grad is None else dtype_code(host_grad.dtype), ptr(finite_flag), ptr(status), nseg,
        ctypes.cast(segments, c_void_p), max_blocks, stream_handle())
    if rc != 0:
        raise RuntimeError(f"ft_rs_adam failed (code {rc})")


def ar_adam(world: int, rank: int, grad_ptrs, flag_ptrs, grad_dtype: torch.dtype, shard: int,
            scale: float, seq: int, reduced_out: Optional[torch.Tensor], do_adam: bool,
            master: torch.Tensor, m: torch.Tensor, v: torch.Tensor, param_ptrs,
            param_dtype: torch.dtype, finite_flag: Optional[torch.Tensor], segments, nseg: int,
            max_blocks: int = 64, start_slot: int = 6, done_slot: int = 7):
    """All-reduce form of the fused kernel for parameters every rank keeps
    whole (``ft_ar_adam`` in ``csrc/comm/rs_adam.cu``): rank ``r`` reduces slice
    ``r`` of all ranks' gradient buffers, updates its slice of the fp32 state
    and stores the new parameters into slice ``r`` of every rank's buffer."""
    rc = _lib().ft_ar_adam(
        world, rank, ctypes.cast(grad_ptrs, c_void_p), ctypes.cast(flag_ptrs, c_void_p) if flag_ptrs
        is not None else None, dtype_code(grad_dtype), shard, float(scale), seq, start_slot, done_slot,
        ptr(reduced_out), int(do_adam), ptr(master), ptr(m), ptr(v), ctypes.cast(param_ptrs, c_void_p),
        dtype_code(param_dtype), ptr(finite_flag), nseg, ctypes.cast(segments, c_void_p), max_blocks,
        stream_handle())
    if rc != 0:
        raise RuntimeError(f"ft_ar_adam failed (code {rc})")


def comm_error() -> int:
    return _lib().ft_comm_error()


# ------------------------------------------------------------ all-gather + GEMM
_AG_DECLARED = False


def _ag_lib():
    global _AG_DECLARED
    lib = cuda_lib()
    if not _AG_DECLARED:
        lib.ft_ag_gemm.argtypes = [c_int, c_int, c_void_p, c_void_p, c_uint32, c_int, c_int, c_int64, c_int64,
                                   c_void_p, c_int64, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int,
                                   c_void_p]
        lib.ft_peer_gather.argtypes = [c_int, c_int, c_void_p, c_void_p, c_uint32, c_int, c_int, c_int64,
                                       c_int, c_void_p]
        lib.ft_peer_gather_range.argtypes = [c_int, c_int, c_void_p, c_void_p, c_uint32, c_int, c_int,
                                             c_int64, c_int64, c_int64, c_int, c_void_p]
        lib.ft_ag_set_spin_budget.argtypes = [ctypes.c_longlong]
        _AG_DECLARED = True
    return lib


AG_GEMM_CHUNK = 8192          # granularity of ownership inside the all-gather GEMM (bytes)


def ag_gemm(world: int, rank: int, buf_ptrs, flag_ptrs, seq: int, x: torch.Tensor, n: int,
            out: Optional[torch.Tensor] = None, w_off_bytes: int = 0, shard_bytes: Optional[int] = None,
            start_slot: int = 2, done_slot: int = 3) -> torch.Tensor:
    """``out[M, n] = x[M, K] @ W.T`` with ``W [n, K]`` gathered inside the same kernel.
    ``buf_ptrs`` are the peer mappings of every rank's flat buffer, sharded in contiguous
    pieces of ``shard_bytes``; ``W`` starts ``w_off_bytes`` into it and the part of it this
    rank owns is in place.  Default: the buffer is ``W`` itself, row-sharded evenly."""
    m, k = x.shape
    if out is None:
        out = torch.empty(m, n, dtype=x.dtype, device=x.device)
    if shard_bytes is None:
        if n % world:
            raise ValueError("a row-sharded weight needs its rows to divide by the world size")
        shard_bytes = n // world * k * x.element_size()
    rc = _ag_lib().ft_ag_gemm(world, rank, ctypes.cast(buf_ptrs, c_void_p),
                              ctypes.cast(flag_ptrs, c_void_p) if flag_ptrs is not None else None, seq,
                              start_slot, done_slot, int(w_off_bytes), int(shard_bytes), ptr(x), x.stride(0),
                              ptr(out), out.stride(0), dtype_code(out.dtype), m, n, k, dtype_code(x.dtype),
                              stream_handle())
    if rc != 0:
        raise RuntimeError(f"ft_ag_gemm failed (code {rc})")
    return out


def ag_gemm_covers(m: int, k: int, w_off_bytes: int, shard_bytes: int) -> bool:
    """Whether ``ft_ag_gemm`` takes this shape and placement."""
    return m > 128 and k % 64 == 0 and w_off_bytes % AG_GEMM_CHUNK == 0 and shard_bytes % AG_GEMM_CHUNK == 0


def set_wait_seconds(seconds: float, device=None):
    """Limit of every cross-GPU wait inside the fused kernels (start / end barriers of the
    reduce kernels, start / end / per-block waits of the gather), converted to SM clock
    cycles at the device's maximum clock.  Applies to kernels launched afterwards."""
    try:
        props = torch.cuda.get_device_properties(device if device is not None else torch.cuda.current_device())
        khz = int(getattr(props, "clock_rate", 0)) or 1_965_000
    except Exception:                                              # the limit matters, its exact length does not
        khz = 1_965_000
    cycles = int(float(seconds) * khz * 1e3)
    lib = _ag_lib()
    lib.ft_comm_set_spin_budget.argtypes = [ctypes.c_longlong]
    lib.ft_comm_set_spin_budget(cycles)
    lib.ft_ag_set_spin_budget(cycles)
    return cycles


def peer_gather(world: int, rank: int, buf_ptrs, flag_ptrs, seq: int, shard_bytes: int,
                num_copiers: int = 16, start_slot: int = 4, done_slot: int = 5):
    """Pull every remote shard of a flat peer-mapped buffer into the local copy."""
    rc = _ag_lib().ft_peer_gather(world, rank, ctypes.cast(buf_ptrs, c_void_p),
                                  ctypes.cast(flag_ptrs, c_void_p), seq, start_slot, done_slot,
                                  shard_bytes, num_copiers, stream_handle())
    if rc != 0:
        raise RuntimeError(f"ft_peer_gather failed (code {rc})")


def peer_gather_range(world: int, rank: int, buf_ptrs, flag_ptrs, seq: int, shard_bytes: int,
                      range_lo: int, range_hi: int, num_copiers: int = 148, start_slot: int = 4,
                      done_slot: int = 5):
    """Pull bytes ``[range_lo, range_hi)`` of a flat peer-mapped buffer from their owners
    (what this rank owns is left alone)."""
    rc = _ag_lib().ft_peer_gather_range(world, rank, ctypes.cast(buf_ptrs, c_void_p),
                                        ctypes.cast(flag_ptrs, c_void_p), seq, start_slot, done_slot,
                                        shard_bytes, range_lo, range_hi, num_copiers, stream_handle())
    if rc != 0:
        raise RuntimeError(f"ft_peer_gather_range failed (code {rc})")
