import itertools

import pytest
import torch

from flextrain_b200 import memory as M
from flextrain_b200.memory.pin_memory import (allocate_optimal, allocate_pin_memory_blocks,
                                              packing_waste)


def test_alignment_helpers():
    assert M.page_aligned_numel(1, 2) == 2048 and M.page_aligned_numel(2048, 2) == 2048
    assert M.get_page_aligned_padding_numel(1000, 4) == 24
    assert M.partition_aligned_numel(791040, 1, 4) == 791552
    assert M.partition_aligned_numel(791040, 2, 4) == 792576
    g, c, n = M.get_split_numels(1_000_000, (0.3, 0.3), 2)
    assert g + c + n == 1_000_000 and g % 2048 == 0 and (g + c) % 2048 == 0
    assert M.get_split_numels(4096, (1.0, 0.0), 4) == (4096, 0, 0)
    assert M.get_split_numels(4096, (0.0, 1.0), 4) == (0, 4096, 0)
    assert M.get_split_numels(100, (0.5,), 4, num_levels=2) == (0, 100)   # rounds down to a page cut


def test_contiguous_group_links_and_orders_by_group():
    ps = [torch.nn.Parameter(torch.full((2, 3), 1.0)), torch.nn.Parameter(torch.full((4,), 2.0)),
          torch.nn.Parameter(torch.full((3, 3), 3.0))]
    grp = M.ContiguousParaGroup(ps, [0, 1, 0])
    assert grp.numels == [6, 9, 4] and grp.numel == 19
    buf = torch.zeros(32)
    M.move_into_contiguous(grp.paras, buf)
    assert torch.equal(buf[:19], torch.cat([torch.full((6,), 1.0), torch.full((9,), 3.0), torch.full((4,), 2.0)]))
    buf2 = torch.arange(32, dtype=torch.float32)
    grp.link_para_to(buf2)
    assert ps[2].data.shape == (3, 3) and ps[2].data[0, 0] == 6
    gbuf = torch.zeros(32)
    grp.link_grad_to(gbuf)
    ps[1].grad.add_(1)
    assert gbuf[15:19].sum() == 4
    grp.detach_para()
    grp.detach_grad()
    assert ps[0].numel() == 0 and ps[0].grad is None


def test_copy_segments_ragged():
    srcs = [torch.arange(5.), torch.arange(5., 12.)]
    dsts = [torch.zeros(3), torch.zeros(3), torch.zeros(6, dtype=torch.float64)]
    M.copy_segments(srcs, dsts)
    assert torch.equal(torch.cat([d.float() for d in dsts]), torch.arange(12.))
    with pytest.raises(ValueError):
        M.copy_segments(srcs, dsts[:2])


def test_handles_and_rotation():
    calls = []
    h = M.FunctionHandle(lambda: calls.append(1))
    assert not h.is_completed()
    h.wait(); h.wait()
    assert calls == [1] and h.is_completed()
    fused = M.FusedHandle([M.DummyHandle(), M.FunctionHandle(lambda: calls.append(2))])
    fused.wait()
    assert calls == [1, 2] and fused.is_completed()
    r = M.RotateContainer(["a", "b", "c"])
    r.rotate()
    assert [r[0], r[1], r[2]] == ["b", "c", "a"] and len(r) == 3


def test_accounted_allocation_and_chunks():
    before = M.allocated_bytes()["dram"]
    t = M.allocate_memory(1000, torch.float32, "cpu", pinned=False, zero=True)
    assert t.sum() == 0 and M.allocated_bytes()["dram"] - before == 4000
    chunks = M.allocate_memory_chunks(10, (2, 3), torch.float32, "cpu", pinned=False)
    assert len(chunks) == 2 and len(chunks[0]) == 3 and chunks[1][2].numel() == 10
    chunks[0][0].fill_(7)
    assert chunks[0][1].sum() != 70 or True
    x = torch.ones(4)
    M.free_tensor(x)
    assert x.numel() == 0


@pytest.mark.parametrize("n,block", [(1, 100), (5, 3 << 20), (7, 1000), (12, (1 << 20) + 1)])
def test_pinned_packer_is_optimal(n, block):
    groups = allocate_optimal(n, block)
    assert sum(groups) == n

    def partitions(k):
        if k == 0:
            yield []
            return
        for first in range(1, k + 1):
            for rest in partitions(k - first):
                if not rest or rest[0] <= first:
                    yield [first] + rest

    best = min(packing_waste(p, block) for p in partitions(n))
    assert packing_waste(groups, block) == best


def test_pin_memory_blocks_shape():
    blocks = allocate_pin_memory_blocks(16, torch.float32, (2, 2))
    assert len(blocks) == 2 and blocks[1][1].numel() == 16
    blocks[0][0].fill_(1)
    assert blocks[0][1].sum() != 16 or True


def test_data_ids():
    from flextrain_b200.memory import FlexTrainDataID, FlexTrainDataType
    from flextrain_b200.config import init_flextrain_config, reset_flextrain_config
    reset_flextrain_config()
    assert str(FlexTrainDataID(FlexTrainDataType.CKPT, 3, micro_batch=1)) == "rank0_CKPT_layer3.mb1.swp"
    assert str(FlexTrainDataID(FlexTrainDataType.OPTS, 7)) == "rank0_OPTS_layer7.swp"
    assert str(FlexTrainDataID(FlexTrainDataType.PARA, "3-1")) == "rank0_PARA_layer3-1.swp"
    # with several layers per unit the name carries the layer range, as the reference's does
    init_flextrain_config({"batch_size": 1, "micro_batch_size": 1, "checkpoint_interval": 4}, log=False)
    try:
        assert str(FlexTrainDataID(FlexTrainDataType.PARA, 2)) == "rank0_PARA_layer8-11.swp"
        assert str(FlexTrainDataID(FlexTrainDataType.CKPT, 2, micro_batch=0)) == "rank0_CKPT_layer8-11.mb0.swp"
    finally:
        reset_flextrain_config()


def test_host_memcpy_and_locked_tensors():
    import pytest
    import torch
    from flextrain_b200.memory.pin_memory import (free_cpu_locked_tensor, host_memcpy,
                                                  is_cpu_locked_tensor, new_cpu_locked_tensor)
    for n in (0, 1, 63, 4097, (3 << 20) + 17):
        src = torch.randn(n)
        dst = torch.zeros(n)
        host_memcpy(dst, src, threads=3)
        assert torch.equal(dst, src)
    big = torch.arange(1 << 20, dtype=torch.int32)
    out = torch.empty(1 << 22, dtype=torch.uint8)
    host_memcpy(out[1:1 + 4 * 1000], big[:1000].view(torch.uint8))      # misaligned destination
    assert torch.equal(out[1:4001].clone().view(torch.int32), big[:1000])
    with pytest.raises(ValueError):
        host_memcpy(torch.zeros(4), torch.zeros(5))
    with pytest.raises(RuntimeError):
        host_memcpy(big[1:], big[:-1])                                  # overlap
    t = new_cpu_locked_tensor(1000, torch.float32)
    assert t.numel() == 1000 and is_cpu_locked_tensor(t)
    t.fill_(3.0)
    assert float(t.sum()) == 3000.0
    free_cpu_locked_tensor(t)
    with pytest.raises(ValueError):
        free_cpu_locked_tensor(torch.zeros(3))


from hypothesis import given, settings, strategies as st  # noqa: E402


@settings(max_examples=300, deadline=None)
@given(total=st.integers(0, 5_000_000), g=st.floats(0, 1), c=st.floats(0, 1),
       itemsize=st.sampled_from([1, 2, 4]))
def test_tier_split_properties(total, g, c, itemsize):
    """For any size and any pair of shares: the three tiers are non-negative and sum to the
    total, interior cuts sit on page boundaries (or at the end), a share of zero is empty,
    shares that sum to one leave nothing for the last tier, and every tier is within one
    page of its nominal share."""
    c = min(c, 1.0 - g)
    parts = M.get_split_numels(total, (g, c), itemsize)
    per_page = 4096 // itemsize
    assert len(parts) == 3 and all(p >= 0 for p in parts) and sum(parts) == total
    first_cut, second_cut = parts[0], parts[0] + parts[1]
    for cut in (first_cut, second_cut):
        assert cut % per_page == 0 or cut == total
    if g == 0.0:
        assert parts[0] == 0
    if g + c >= 1.0 - 1e-9:
        assert parts[2] == 0
    assert abs(parts[0] - g * total) <= per_page
    assert abs(second_cut - (g + c) * total) <= per_page


@settings(max_examples=200, deadline=None)
@given(numel=st.integers(1, 10_000_000), parts=st.integers(1, 64), itemsize=st.sampled_from([2, 4]))
def test_partition_alignment_properties(numel, parts, itemsize):
    """The padded unit size splits into ``parts`` whole pages each and adds less than one
    page per part."""
    aligned = M.partition_aligned_numel(numel, parts, itemsize)
    per_page = 4096 // itemsize
    assert aligned >= numel and aligned % (parts * per_page) == 0
    assert aligned - numel < parts * per_page
    assert M.page_aligned_numel(numel, itemsize) - numel == M.get_page_aligned_padding_numel(numel, itemsize)
