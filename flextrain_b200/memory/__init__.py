"""Memory primitives shared by the coordinators.

Parity: flextrain/memory/__init__.py:1-412 - data ids and swap-file names
:20-49, ``free_tensor`` :52-60, ``move_into_contiguous`` :63-84,
``copy_segments`` :87-135, ``ContiguousParaGroup`` :138-184, waitable handles
:187-237, ``RotateContainer`` :240-248, accounted allocation :251-312 and the
alignment helpers :315-363.  The single side stream of the reference
(``FlexTrainDataStream`` :366-412) is replaced by the event-ordered stream set
of ``utils/device.py``; ``get_data_stream`` returns that set.
"""
from __future__ import annotations

import ctypes
import os
import threading
from dataclasses import dataclass
from enum import Enum
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from ..defaults import PAGE_SIZE
from ..utils import distributed as dist
from ..utils.device import StreamSet, get_streams
from ..utils.logging import rank0_logger


# ---------------------------------------------------------------- data ids
class FlexTrainDataType(Enum):
    CKPT = 0
    PARA = 1
    GRAD = 2
    OPTS = 3


@dataclass(frozen=True)
class FlexTrainDataID:
    """Names one swappable object of a unit; ``str()`` is its swap-file name.  As in the
    reference (flextrain/memory/__init__.py:40-49) a unit is named by the layers it holds:
    ``rank{r}_{TYPE}_layer{i}.swp`` with one layer per unit, ``..._layer{first}-{last}.swp`` with
    ``checkpoint_interval`` > 1.  Objects that exist once per micro-batch (activation
    checkpoints) carry ``.mb{j}`` in addition, which the reference has no need for because
    it packs a unit's micro-batches into one file.  A string is used as the layer part as is."""
    data_type: FlexTrainDataType
    unit_index: object           # unit number, or a ready-made layer label
    micro_batch: Optional[int] = None

    def layer_label(self) -> str:
        if not isinstance(self.unit_index, int):
            return str(self.unit_index)
        interval = 1
        try:
            from ..config import get_flextrain_config
            interval = int(get_flextrain_config().checkpoint_interval)
        except RuntimeError:
            pass
        first = self.unit_index * interval
        return f"{first}-{first + interval - 1}" if interval > 1 else str(first)

    def __str__(self):
        mb = "" if self.micro_batch is None else f".mb{self.micro_batch}"
        return f"rank{dist.get_rank()}_{self.data_type.name}_layer{self.layer_label()}{mb}.swp"


# ------------------------------------------------------------------ handles
class Waitable:
    def wait(self):
        raise NotImplementedError

    def is_completed(self) -> bool:
        raise NotImplementedError


class DummyHandle(Waitable):
    def wait(self):
        return None

    def is_completed(self):
        return True


class FunctionHandle(Waitable):
    """Runs ``fn`` once, at the first ``wait``."""

    def __init__(self, fn: Callable[[], None]):
        self._fn = fn

    def wait(self):
        fn, self._fn = self._fn, None
        if fn is not None:
            fn()

    def is_completed(self):
        return self._fn is None


class EventHandle(Waitable):
    """Completion of GPU work up to a recorded event."""

    def __init__(self, event):
        self._event = event

    def wait(self):
        self._event.synchronize()

    def is_completed(self):
        return self._event.query()


class FutureHandle(Waitable):
    """Completion of a ``concurrent.futures.Future`` (host worker threads)."""

    def __init__(self, future):
        self._future = future

    def wait(self):
        return self._future.result()

    def is_completed(self):
        return self._future.done()


class FusedHandle(Waitable):
    def __init__(self, handles: Iterable[Waitable]):
        self._handles = list(handles)

    def wait(self):
        for h in self._handles:
            h.wait()
        self._handles = []

    def is_completed(self):
        return all(h.is_completed() for h in self._handles)


class RotateContainer:
    """Fixed ring of buffers; ``rotate`` advances which one is at index 0."""

    def __init__(self, items: Sequence):
        self._items = list(items)

    def __getitem__(self, i):
        return self._items[i]

    def __setitem__(self, i, v):
        self._items[i] = v

    def __len__(self):
        return len(self._items)

    def rotate(self):
        self._items.append(self._items.pop(0))


# --------------------------------------------------------------- alignment
def page_aligned_numel(numel: int, itemsize: int, page: int = PAGE_SIZE) -> int:
    """Smallest element count >= ``numel`` whose byte size is a page multiple."""
    per_page = page // itemsize
    return -(-numel // per_page) * per_page


def get_page_aligned_padding_numel(numel: int, itemsize: int) -> int:
    return page_aligned_numel(numel, itemsize) - numel


def partition_aligned_numel(numel: int, parts: int, itemsize: int, page: int = PAGE_SIZE) -> int:
    """Smallest count >= ``numel`` that splits into ``parts`` page-sized-multiple
    pieces (flextrain/memory/__init__.py:322-323)."""
    quantum = parts * (page // itemsize)
    return -(-numel // quantum) * quantum


def get_split_numels(total: int, ratios: Sequence[float], itemsize: int,
                     num_levels: int = 3, page: int = PAGE_SIZE) -> Tuple[int, ...]:
    """Cut ``total`` elements into ``num_levels`` consecutive tiers.  ``ratios``
    gives the share of every tier but the last; interior cut points are rounded
    to page boundaries and the last tier takes what is left."""
    per_page = max(1, page // itemsize)
    ratios = list(ratios)[: num_levels - 1]
    ratios += [0.0] * (num_levels - 1 - len(ratios))
    out, used, acc = [], 0, 0.0
    for r in ratios:
        acc += r
        cut = min(total, int(round(acc * total / per_page)) * per_page)
        if acc >= 1.0 - 1e-9:
            cut = total            # a full share is a full share, also for tensors smaller than a page
        cut = max(cut, used)
        out.append(cut - used)
        used = cut
    out.append(total - used)
    return tuple(out)


# -------------------------------------------------------------- allocation
class _Accounting:
    def __init__(self):
        self.lock = threading.Lock()
        self.bytes: Dict[str, int] = {"hbm": 0, "pinned": 0, "dram": 0}

    def add(self, kind: str, nbytes: int):
        with self.lock:
            self.bytes[kind] += nbytes


_ACCOUNT = _Accounting()
_PINNED_KEEPALIVE: List[object] = []


def allocated_bytes() -> Dict[str, int]:
    return dict(_ACCOUNT.bytes)


def _pinned_exact(nbytes: int) -> torch.Tensor:
    """Exact-size page-locked allocation from the native pool (PyTorch's pinned
    allocator rounds every request up to a power of two, which wastes up to
    half of a large buffer)."""
    from ..ops.native import cuda_lib
    lib = cuda_lib()
    addr = lib.ft_pinned_alloc(ctypes.c_size_t(max(nbytes, 1)))
    if not addr:
        raise MemoryError(f"page-locked allocation of {nbytes} bytes failed")
    buf = (ctypes.c_uint8 * max(nbytes, 1)).from_address(addr)
    t = torch.frombuffer(buf, dtype=torch.uint8, count=max(nbytes, 1))
    _PINNED_KEEPALIVE.append(buf)
    return t[:nbytes]


# Guard mode (environment variable FLEXTRAIN_GUARD=1, a debugging aid): every buffer from
# ``allocate_memory`` gets a band of pattern bytes on both sides, ``check_guards()`` reports
# every band that no longer holds the pattern.  A copy, kernel or host routine that runs past
# the end of a tier buffer, a staging buffer or a ring slot is then seen at the end of the
# step that did it instead of as wrong numbers many steps later.  The bands keep the
# alignment of the payload (one page on the host, 512 bytes on the device).
_GUARD_BYTE = 0xA5
_GUARDS: List[tuple] = []          # (whole uint8 view, band bytes, payload bytes, where allocated)


def guard_mode() -> bool:
    return os.environ.get("FLEXTRAIN_GUARD", "0") not in ("", "0")


def _guarded(numel: int, dtype: torch.dtype, device, pinned: bool, zero: bool, itemsize: int) -> torch.Tensor:
    import sys
    band = 512 if torch.device(device).type == "cuda" else PAGE_SIZE
    nbytes = numel * itemsize
    padded = (nbytes + band - 1) // band * band
    whole = _allocate(2 * band + padded, torch.uint8, device, pinned, False, account=nbytes)
    whole[:band].fill_(_GUARD_BYTE)
    whole[band + nbytes:].fill_(_GUARD_BYTE)
    frame = sys._getframe(2)
    where = f"{os.path.basename(frame.f_code.co_filename)}:{frame.f_lineno} ({frame.f_code.co_name})"
    _GUARDS.append((whole, band, nbytes, where))
    t = whole[band:band + nbytes].view(dtype)
    return t.zero_() if zero else t


def check_guards(raise_on_damage: bool = True) -> List[str]:
    """Guard mode: the buffers whose bands were written to, as ``where allocated: which side,
    first damaged byte``.  Synchronises the device first.  Empty list when all is well (and
    always outside guard mode)."""
    if not _GUARDS:
        return []
    if torch.cuda.is_available() and any(w.is_cuda for w, _, _, _ in _GUARDS):
        torch.cuda.synchronize()
    damaged = []
    for whole, band, nbytes, where in _GUARDS:
        for side, piece, base in (("before", whole[:band], -band), ("after", whole[band + nbytes:], nbytes)):
            bad = (piece != _GUARD_BYTE).nonzero()
            if bad.numel():
                damaged.append(f"{where}: {nbytes} bytes, band {side} the buffer written at byte offset "
                               f"{base + int(bad[0])} ({int(bad.numel())} bytes differ)")
    if damaged and raise_on_damage:
        raise RuntimeError("buffer overrun: " + "; ".join(damaged))
    return damaged


def clear_guards():
    _GUARDS.clear()


def allocate_memory(numel: int, dtype: torch.dtype, device, pinned: bool = True,
                    zero: bool = False) -> torch.Tensor:
    """Accounted flat allocation.  ``device`` cpu + ``pinned`` gives exact-size
    page-locked memory when CUDA is in use, plain memory otherwise."""
    itemsize = torch.empty((), dtype=dtype).element_size()
    if guard_mode() and numel > 0:
        return _guarded(numel, dtype, device, pinned, zero, itemsize)
    return _allocate(numel, dtype, device, pinned, zero)


def _allocate(numel: int, dtype: torch.dtype, device, pinned: bool, zero: bool,
              account: Optional[int] = None) -> torch.Tensor:
    device = torch.device(device)
    itemsize = torch.empty((), dtype=dtype).element_size()
    nbytes = numel * itemsize
    booked = nbytes if account is None else account     # guard bands are not booked
    if device.type == "cuda":
        _ACCOUNT.add("hbm", booked)
        t = torch.empty(numel, dtype=dtype, device=device)
        return t.zero_() if zero else t
    if pinned and dist.is_cuda() and numel > 0:
        _ACCOUNT.add("pinned", booked)
        try:
            t = _pinned_exact(nbytes).view(dtype)
        except Exception:
            t = torch.empty(numel, dtype=dtype).pin_memory()
        return t.zero_() if zero else t
    _ACCOUNT.add("dram", booked)
    return torch.zeros(numel, dtype=dtype) if zero else torch.empty(numel, dtype=dtype)


def allocate_memory_chunks(numel: int, chunks, dtype: torch.dtype, device,
                           pinned: bool = True, zero: bool = False):
    """``chunks`` (an int or a tuple of ints) equal flat buffers, returned as
    nested lists; they are carved from one allocation."""
    if isinstance(chunks, int):
        chunks = (chunks,)
    total = 1
    for c in chunks:
        total *= c
    flat = allocate_memory(numel * total, dtype, device, pinned, zero)

    def carve(level, offset):
        if level == len(chunks):
            return flat[offset * numel:(offset + 1) * numel]
        stride = 1
        for c in chunks[level + 1:]:
            stride *= c
        return [carve(level + 1, offset + i * stride) for i in range(chunks[level])]

    return carve(0, 0)


class _Traffic:
    """Bytes moved between tiers since the last ``reset`` (host-side counters:
    ``h2d``, ``d2h``, ``d2d``, ``h2h`` copies, ``nvme_read`` / ``nvme_write``,
    ``gather`` / ``reduce`` collective payloads)."""

    KINDS = ("h2d", "d2h", "d2d", "h2h", "nvme_read", "nvme_write", "gather", "reduce")

    def __init__(self):
        self.lock = threading.Lock()
        self.bytes: Dict[str, int] = {k: 0 for k in self.KINDS}

    def add(self, kind: str, nbytes: int):
        with self.lock:
            self.bytes[kind] = self.bytes.get(kind, 0) + int(nbytes)

    def snapshot(self, reset: bool = False) -> Dict[str, int]:
        with self.lock:
            out = dict(self.bytes)
            if reset:
                for k in self.bytes:
                    self.bytes[k] = 0
        return out


TRAFFIC = _Traffic()


def tier_copy(dst: torch.Tensor, src: torch.Tensor, non_blocking: bool = True) -> torch.Tensor:
    """``dst.copy_(src)`` that also books the bytes under the pair of tiers it
    crosses (the engine's per-tier traffic counters)."""
    kind = ("d" if src.is_cuda else "h") + "2" + ("d" if dst.is_cuda else "h")
    TRAFFIC.add(kind, dst.numel() * dst.element_size())
    return dst.copy_(src, non_blocking=non_blocking)


def free_tensor(t: torch.Tensor, record_stream: bool = False):
    """Release ``t``'s storage while the Python object stays alive."""
    if record_stream and t.is_cuda:
        t.record_stream(torch.cuda.current_stream())
    t.data = torch.empty(0, dtype=t.dtype, device=t.device)


def move_into_contiguous(srcs: Iterable[torch.Tensor], dst: torch.Tensor):
    """Copy every tensor of ``srcs`` back to back into flat ``dst`` and re-point
    each source's ``.data`` at its new home."""
    offset = 0
    for s in srcs:
        n = s.numel()
        view = dst[offset:offset + n].view(s.shape)
        view.copy_(s.data, non_blocking=True)
        s.data = view
        offset += n
    return offset


def copy_segments(srcs: Sequence[torch.Tensor], dsts: Sequence[torch.Tensor]):
    """Ragged copy: the concatenation of ``srcs`` is written over the
    concatenation of ``dsts`` (flat tensors; dtype conversion allowed)."""
    if sum(s.numel() for s in srcs) != sum(d.numel() for d in dsts):
        raise ValueError("copy_segments: source and destination sizes differ")
    si = di = so = do = 0
    while si < len(srcs) and di < len(dsts):
        s, d = srcs[si], dsts[di]
        n = min(s.numel() - so, d.numel() - do)
        if n:
            d[do:do + n].copy_(s[so:so + n], non_blocking=True)
        so += n
        do += n
        if so == s.numel():
            si, so = si + 1, 0
        if do == d.numel():
            di, do = di + 1, 0


class ContiguousParaGroup:
    """The parameters of one unit in their flat order.

    Parameters with equal ``grouping`` id are made adjacent (stable order inside
    a group), so every optimizer param group covers few contiguous ranges.
    ``link_para_to(buffer)`` points every parameter's ``.data`` at its slice of
    a flat buffer; ``link_grad_to`` does the same for ``.grad``; ``detach_*``
    drop the views again so the buffer can be reused.
    """

    def __init__(self, params: Sequence[torch.nn.Parameter],
                 grouping: Optional[Sequence[int]] = None):
        params = list(params)
        if grouping is None:
            grouping = [0] * len(params)
        order = sorted(range(len(params)), key=lambda i: (grouping[i], i))
        self.paras = [params[i] for i in order]
        self.grouping = [grouping[i] for i in order]
        self.shapes = [tuple(p.shape) for p in self.paras]
        self.numels = [p.numel() for p in self.paras]
        self.numel = sum(self.numels)
        self.offsets = [0]
        for n in self.numels:
            self.offsets.append(self.offsets[-1] + n)

    def link_para_to(self, buffer: torch.Tensor):
        for p, off, n, shape in zip(self.paras, self.offsets, self.numels, self.shapes):
            p.data = buffer[off:off + n].view(shape)

    def link_grad_to(self, buffer: torch.Tensor):
        for p, off, n, shape in zip(self.paras, self.offsets, self.numels, self.shapes):
            p.grad = buffer[off:off + n].view(shape)

    def detach_para(self):
        for p in self.paras:
            p.data = torch.empty(0, dtype=p.dtype, device=p.device)

    def detach_grad(self):
        for p in self.paras:
            p.grad = None


def get_data_stream() -> StreamSet:
    """The rank's stream set (compute / h2d / d2h / opt)."""
    return get_streams()


# ------------------------------------------------- names of the reference module
# flextrain/memory/__init__.py spells these helpers with a ``get_`` prefix and keeps two
# module-level byte counters; scripts written against it find the same names here.
get_page_aligned_numel = page_aligned_numel
get_partition_aligned_numel = partition_aligned_numel
FlexTrainDataStream = StreamSet


def get_allocated_dram_size() -> int:
    """Bytes of host memory handed out so far, pinned and pageable (flextrain/memory/__init__.py:307-308)."""
    return _ACCOUNT.bytes["pinned"] + _ACCOUNT.bytes["dram"]


def get_allocated_vram_size() -> int:
    """Bytes of device memory handed out so far (flextrain/memory/__init__.py:311-312)."""
    return _ACCOUNT.bytes["hbm"]


def __getattr__(name):
    # AsyncIOHandle lives with the NVMe engine, which itself imports this module
    if name == "AsyncIOHandle":
        from .nvme_swapper import AsyncIOHandle
        return AsyncIOHandle
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
