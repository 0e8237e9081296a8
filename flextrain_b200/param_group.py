"""Interval algebra that maps optimizer param groups onto flat unit buffers.

Parity: flextrain/param_group.py:1-477 - ``GroupSegment``/``StepContext``
:22-35, ``merge_segments``/``create_group_segments``/``slice_segments`` :42-175,
``create_step_contexts`` :178-224, the cut-plan helpers :227-362 and
``StepContextContainer`` :365-477.

A unit's parameters are flattened into one buffer.  Each element belongs to one
optimizer param group (its own lr / weight decay).  The buffer is then cut by
several independent partitions - rank shards, memory tiers, the alpha split,
per-micro-batch chunks, staging-buffer capacities - and the Adam kernels need,
for every resulting piece, the group it belongs to and views of the matching
master / gradient / state / device-copy buffers.  Everything here works on
half-open integer ranges, so it is testable without tensors.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch


@dataclass(frozen=True)
class GroupSegment:
    """Elements ``[start, end)`` of a flat buffer belong to param group ``group``."""
    group: int
    start: int
    end: int

    @property
    def numel(self) -> int:
        return self.end - self.start

    def shifted(self, delta: int) -> "GroupSegment":
        return GroupSegment(self.group, self.start + delta, self.end + delta)


@dataclass
class StepContext:
    """One contiguous Adam call: the group's hyper-parameters and flat views of
    the same element range in every buffer that takes part."""
    group: Dict
    master: torch.Tensor
    grad: torch.Tensor
    states: List[torch.Tensor]
    device_copy: Optional[torch.Tensor] = None
    group_index: int = -1

    @property
    def numel(self) -> int:
        return self.master.numel()


def merge_segments(segments: Iterable[GroupSegment]) -> List[GroupSegment]:
    """Drop empty segments and fuse neighbours that touch and share a group."""
    out: List[GroupSegment] = []
    for seg in segments:
        if seg.end <= seg.start:
            continue
        if out and out[-1].group == seg.group and out[-1].end == seg.start:
            out[-1] = GroupSegment(seg.group, out[-1].start, seg.end)
        else:
            out.append(seg)
    return out


def create_group_segments(numels: Sequence[int], groups: Sequence[int],
                          offset: int = 0) -> List[GroupSegment]:
    """Segments of a buffer that concatenates tensors of ``numels`` elements
    whose param-group indices are ``groups``."""
    if len(numels) != len(groups):
        raise ValueError("numels and groups must have equal length")
    segs, cursor = [], offset
    for n, g in zip(numels, groups):
        segs.append(GroupSegment(int(g), cursor, cursor + int(n)))
        cursor += int(n)
    return merge_segments(segs)


def slice_segments(segments: Sequence[GroupSegment], start: int, end: int,
                   rebase: bool = True) -> List[GroupSegment]:
    """The part of ``segments`` inside ``[start, end)``; with ``rebase`` the
    result is expressed relative to ``start``."""
    out = []
    for seg in segments:
        lo, hi = max(seg.start, start), min(seg.end, end)
        if lo < hi:
            shift = -start if rebase else 0
            out.append(GroupSegment(seg.group, lo + shift, hi + shift))
    return merge_segments(out)


def segments_numel(segments: Iterable[GroupSegment]) -> int:
    return sum(s.numel for s in segments)


def merge_slice_plans(*plans: Sequence[int]) -> List[int]:
    """Union of several cut-point lists (each a sorted list of offsets that
    starts at the region start and ends at the region end)."""
    cuts = set()
    for plan in plans:
        cuts.update(int(c) for c in plan)
    return sorted(cuts)


def even_slice_plan(start: int, end: int, parts: int, align: int = 1) -> List[int]:
    """Cut ``[start, end)`` into ``parts`` nearly equal pieces whose interior
    boundaries are multiples of ``align`` relative to ``start``."""
    total = end - start
    cuts = [start]
    for i in range(1, parts):
        c = (total * i // parts) // align * align
        cuts.append(start + c)
    cuts.append(end)
    return sorted(set(cuts))


def capacity_slice_plan(start: int, end: int, capacity: int) -> List[int]:
    """Cut ``[start, end)`` into pieces of at most ``capacity`` elements."""
    if capacity <= 0:
        raise ValueError("capacity must be positive")
    cuts = list(range(start, end, capacity))
    cuts.append(end)
    if not cuts or cuts[0] != start:
        cuts.insert(0, start)
    return sorted(set(cuts))


def segment_slice_plan(segments: Sequence[GroupSegment]) -> List[int]:
    cuts = set()
    for s in segments:
        cuts.add(s.start)
        cuts.add(s.end)
    return sorted(cuts)


def ranges_from_plan(plan: Sequence[int]) -> List[Tuple[int, int]]:
    return [(a, b) for a, b in zip(plan[:-1], plan[1:]) if b > a]


def create_tensor_split_plans(tensor_numels: Sequence[int], plan: Sequence[int]) -> List[List[int]]:
    """Distribute one cut-point list over consecutive buffers.

    ``tensor_numels`` are the sizes of buffers laid end to end from ``plan[0]``
    to ``plan[-1]``; the result gives, per non-empty buffer, the lengths of the
    pieces the plan cuts it into.  Every buffer boundary must itself be a cut
    point (merge the boundaries into the plan first).  Counterpart of
    flextrain/param_group.py:267-310, expressed on offsets instead of lengths."""
    numels = [int(n) for n in tensor_numels if n > 0]
    ranges = ranges_from_plan(plan)
    if not numels:
        if ranges:
            raise ValueError("plan covers elements but there is no buffer")
        return []
    if sum(numels) != plan[-1] - plan[0]:
        raise ValueError("buffers and plan cover different numbers of elements")
    out: List[List[int]] = []
    it = iter(ranges)
    for n in numels:
        left, pieces = n, []
        while left > 0:
            a, b = next(it)
            if b - a > left:
                raise ValueError("a buffer boundary is not a cut point of the plan")
            pieces.append(b - a)
            left -= b - a
        out.append(pieces)
    return out


def get_sliced_tensors(tensors, split_plans: Sequence[Sequence[int]]) -> List[torch.Tensor]:
    """Views of flat ``tensors`` (one tensor or a list; empty ones are skipped)
    cut by the per-buffer piece lengths of ``create_tensor_split_plans``
    (flextrain/param_group.py:313-329)."""
    if isinstance(tensors, torch.Tensor):
        tensors = [tensors]
    tensors = [t for t in tensors if t.numel() > 0]
    if len(tensors) != len(split_plans):
        raise ValueError(f"{len(tensors)} buffers but {len(split_plans)} split plans")
    out: List[torch.Tensor] = []
    for t, pieces in zip(tensors, split_plans):
        if t.numel() != sum(pieces):
            raise ValueError(f"pieces {list(pieces)} do not cover a buffer of {t.numel()} elements")
        out.extend(torch.split(t, list(pieces)))
    return out


def create_step_contexts(param_groups: Sequence[Dict], segments: Sequence[GroupSegment],
                         master: torch.Tensor, grad: torch.Tensor,
                         states: Sequence[torch.Tensor],
                         device_copy: Optional[torch.Tensor] = None,
                         base: int = 0) -> List[StepContext]:
    """One ``StepContext`` per segment.  All buffers are flat and cover the same
    element range, which starts at ``base`` in segment coordinates."""
    ctxs = []
    for seg in segments:
        lo, hi = seg.start - base, seg.end - base
        ctxs.append(StepContext(
            group=param_groups[seg.group], group_index=seg.group,
            master=master[lo:hi], grad=grad[lo:hi],
            states=[s[lo:hi] for s in states],
            device_copy=None if device_copy is None else device_copy[lo:hi]))
    return ctxs


def group_step_contexts(contexts: Iterable[StepContext]) -> Dict[int, List[StepContext]]:
    """Bucket contexts by param-group index (one hyper-parameter set each)."""
    out: Dict[int, List[StepContext]] = {}
    for c in contexts:
        out.setdefault(c.group_index, []).append(c)
    return out


@dataclass
class _Piece:
    start: int
    end: int
    segments: List[GroupSegment] = field(default_factory=list)


class StepContextContainer:
    """Cut plan for one region ``[start, end)`` of a flat unit shard.

    The region is intersected with (a) an even split into ``chunks`` pieces
    (one per micro-batch, so host Adam work can be spread over the unit's
    micro-batches), (b) the param-group boundaries and (c) any number of extra
    boundary lists (tier cuts, staging-buffer capacities).  ``plan`` binds flat
    buffers that cover the region; ``container[i]`` then yields the contexts of
    chunk ``i``.  The union of all chunks covers the region exactly once.
    """

    def __init__(self, param_groups: Sequence[Dict], segments: Sequence[GroupSegment],
                 start: int, end: int, chunks: int = 1, align: int = 1,
                 extra_plans: Sequence[Sequence[int]] = ()):
        self.param_groups = param_groups
        self.start, self.end = int(start), int(end)
        self.chunks = max(1, int(chunks))
        self._segments = slice_segments(segments, self.start, self.end, rebase=False)
        chunk_plan = even_slice_plan(self.start, self.end, self.chunks, align)
        # chunk boundaries may coincide when the region is tiny: keep positions
        self._chunk_bounds = [self.start]
        total = self.end - self.start
        for i in range(1, self.chunks):
            self._chunk_bounds.append(self.start + (total * i // self.chunks) // align * align)
        self._chunk_bounds.append(self.end)
        clipped = [[c for c in plan if self.start <= c <= self.end] for plan in extra_plans]
        self._plan = merge_slice_plans(chunk_plan, segment_slice_plan(self._segments),
                                       [self.start, self.end], *clipped)
        self._bound = None

    @property
    def cut_plan(self) -> List[int]:
        return list(self._plan)

    def chunk_range(self, i: int) -> Tuple[int, int]:
        return self._chunk_bounds[i], self._chunk_bounds[i + 1]

    def chunk_pieces(self, i: int) -> List[GroupSegment]:
        lo, hi = self.chunk_range(i)
        out = []
        for a, b in ranges_from_plan(self._plan):
            if a >= lo and b <= hi:
                out.extend(slice_segments(self._segments, a, b, rebase=False))
        return out

    def plan(self, master: torch.Tensor, grad: torch.Tensor, states: Sequence[torch.Tensor],
             device_copy: Optional[torch.Tensor] = None):
        n = self.end - self.start
        for t in (master, grad, *states):
            if t.numel() != n:
                raise ValueError(f"buffer of {t.numel()} elements does not cover the region of {n}")
        if device_copy is not None and device_copy.numel() != n:
            raise ValueError("device copy does not cover the region")
        self._bound = (master, grad, list(states), device_copy)
        return self

    def __len__(self):
        return self.chunks

    def __getitem__(self, i: int) -> List[StepContext]:
        if self._bound is None:
            raise RuntimeError("plan(...) must bind buffers before contexts are requested")
        master, grad, states, device_copy = self._bound
        return create_step_contexts(self.param_groups, self.chunk_pieces(i), master, grad,
                                    states, device_copy, base=self.start)

    def all_contexts(self) -> List[StepContext]:
        out = []
        for i in range(self.chunks):
            out.extend(self[i])
        return out


# ------------------------------------------------------- nested-list helpers
def reshape_list(items: Sequence, shape: Sequence[int]):
    """Flat sequence -> numpy object array of ``shape`` (flextrain/param_group.py:9-10); used
    to address buffers by (unit, micro-batch, ...) index tuples."""
    import numpy as np
    out = np.empty(len(items), dtype=object)
    for i, item in enumerate(items):
        out[i] = item                                   # element-wise: tensors must not be unpacked
    return out.reshape(tuple(shape))


def flatten_list(nested) -> List:
    """Arbitrarily nested lists -> one flat list, depth first (flextrain/param_group.py:13-19)."""
    if not isinstance(nested, list):
        return [nested]
    flat: List = []
    for item in nested:
        flat.extend(flatten_list(item))
    return flat


def is_same_param_group(a, b) -> bool:
    """Param groups are compared by identity, not by value: two groups with equal
    hyper-parameters are still stepped separately (flextrain/param_group.py:38-39)."""
    return a is b
