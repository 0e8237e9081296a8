import torch
from hypothesis import given, settings, strategies as st

from flextrain_b200.param_group import (GroupSegment, StepContextContainer, capacity_slice_plan,
                                        create_group_segments, create_step_contexts, even_slice_plan,
                                        merge_segments, merge_slice_plans, ranges_from_plan,
                                        segments_numel, slice_segments)


def test_merge_and_create():
    segs = create_group_segments([4, 6, 2, 8], [0, 0, 1, 0])
    assert segs == [GroupSegment(0, 0, 10), GroupSegment(1, 10, 12), GroupSegment(0, 12, 20)]
    assert merge_segments([GroupSegment(0, 0, 0), GroupSegment(1, 0, 3), GroupSegment(1, 3, 5)]) == \
        [GroupSegment(1, 0, 5)]


def test_slice_rebase():
    segs = create_group_segments([10, 10, 10], [0, 1, 0])
    assert slice_segments(segs, 5, 25) == [GroupSegment(0, 0, 5), GroupSegment(1, 5, 15), GroupSegment(0, 15, 20)]
    assert slice_segments(segs, 5, 25, rebase=False)[0] == GroupSegment(0, 5, 10)
    assert slice_segments(segs, 30, 40) == []


@settings(max_examples=80, deadline=None)
@given(st.lists(st.tuples(st.integers(1, 50), st.integers(0, 2)), min_size=1, max_size=12),
       st.integers(0, 100), st.integers(0, 100))
def test_slice_covers_exactly_the_requested_range(parts, a, b):
    segs = create_group_segments([p[0] for p in parts], [p[1] for p in parts])
    total = segments_numel(segs)
    lo, hi = sorted((a % (total + 1), b % (total + 1)))
    out = slice_segments(segs, lo, hi, rebase=False)
    assert segments_numel(out) == hi - lo
    for x, y in zip(out[:-1], out[1:]):
        assert x.end == y.start and x.group != y.group
    # every element keeps its group
    owner = {}
    for s in segs:
        for i in range(s.start, s.end):
            owner[i] = s.group
    for s in out:
        assert all(owner[i] == s.group for i in range(s.start, s.end))


def test_plans():
    assert even_slice_plan(0, 100, 4) == [0, 25, 50, 75, 100]
    assert even_slice_plan(0, 100, 3, align=8) == [0, 32, 64, 100]
    assert capacity_slice_plan(10, 35, 10) == [10, 20, 30, 35]
    assert merge_slice_plans([0, 50, 100], [0, 25, 100]) == [0, 25, 50, 100]
    assert ranges_from_plan([0, 5, 5, 9]) == [(0, 5), (5, 9)]


@settings(max_examples=60, deadline=None)
@given(st.lists(st.tuples(st.integers(1, 40), st.integers(0, 1)), min_size=1, max_size=8),
       st.integers(1, 5), st.lists(st.integers(0, 400), max_size=4))
def test_container_chunks_tile_the_region_once(parts, chunks, cuts):
    segs = create_group_segments([p[0] for p in parts], [p[1] for p in parts])
    total = segments_numel(segs)
    start, end = total // 5, total
    groups = [{"lr": 1.0}, {"lr": 2.0}]
    cont = StepContextContainer(groups, segs, start, end, chunks=chunks,
                                extra_plans=[[start] + sorted(c % (total + 1) for c in cuts) + [end]])
    n = end - start
    master = torch.arange(n, dtype=torch.float32)
    cont.plan(master, torch.zeros(n), [torch.zeros(n), torch.zeros(n)], torch.zeros(n))
    seen = torch.zeros(n)
    for i in range(len(cont)):
        for ctx in cont[i]:
            seen[ctx.master.long()] += 1
            assert ctx.group is groups[ctx.group_index]
            assert ctx.grad.numel() == ctx.numel == ctx.states[0].numel() == ctx.device_copy.numel()
    assert torch.all(seen == 1)


def test_step_contexts_bind_views():
    segs = [GroupSegment(0, 10, 14), GroupSegment(1, 14, 20)]
    master = torch.arange(10, dtype=torch.float32)
    ctxs = create_step_contexts([{"a": 1}, {"a": 2}], segs, master, master.clone(), [master.clone()],
                                None, base=10)
    assert [c.numel for c in ctxs] == [4, 6]
    ctxs[1].master.add_(100)
    assert master[4].item() == 104.0


def test_tensor_split_plans_and_sliced_tensors():
    import pytest
    import torch
    from flextrain_b200.param_group import (create_tensor_split_plans, get_sliced_tensors,
                                            merge_slice_plans)
    plan = merge_slice_plans([0, 10, 30], [0, 6, 10, 24, 30])
    plans = create_tensor_split_plans([10, 0, 20], plan)
    assert plans == [[6, 4], [14, 6]]
    bufs = [torch.arange(10.), torch.empty(0), torch.arange(10., 30.)]
    views = get_sliced_tensors(bufs, plans)
    assert [v.numel() for v in views] == [6, 4, 14, 6]
    assert torch.equal(torch.cat(views), torch.arange(30.))
    views[2][0] = -1.0                      # views, not copies
    assert bufs[2][0] == -1.0
    assert create_tensor_split_plans([0, 0], [0]) == []
    with pytest.raises(ValueError):
        create_tensor_split_plans([12, 18], plan)      # 12 is not a cut point
    with pytest.raises(ValueError):
        get_sliced_tensors(bufs[0], plans)
