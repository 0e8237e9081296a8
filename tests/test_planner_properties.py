"""Properties of the closed-form tier planner over random model shapes and machines."""
import types

from hypothesis import given, settings, strategies as st

from flextrain_b200 import planner

GiB = float(1 << 30)


def _shape(layers, hidden, heads, kv_heads, ffn_mult, vocab, mbs, seq):
    head_dim = hidden // heads
    kv = kv_heads * head_dim
    ffn = int(hidden * ffn_mult) // 8 * 8
    layer = 2 * hidden + hidden * (hidden + 2 * kv) + hidden * hidden + 3 * hidden * ffn
    cfg = types.SimpleNamespace(num_layers=layers, layer_numel=layer,
                                total_numel=layers * layer + 2 * vocab * hidden + hidden, hidden=hidden,
                                ffn=ffn, vocab=vocab, seq_len=seq, num_heads=heads, num_kv_heads=kv_heads,
                                head_dim=head_dim)
    return planner.shape_of(cfg, mbs)


shapes = st.builds(_shape, layers=st.integers(2, 96), hidden=st.sampled_from([1024, 2048, 4096, 8192]),
                   heads=st.sampled_from([8, 16, 32, 64]), kv_heads=st.sampled_from([1, 2, 8]),
                   ffn_mult=st.sampled_from([2.6875, 3.5, 4.0]), vocab=st.sampled_from([32000, 128256]),
                   mbs=st.integers(1, 8), seq=st.sampled_from([1024, 4096]))


@settings(max_examples=150, deadline=None)
@given(shape=shapes, world=st.sampled_from([1, 2, 4, 8]), mbpr=st.integers(1, 4),
       hbm=st.floats(20, 180), dram=st.floats(0, 400), nvme=st.floats(0, 2000))
def test_a_plan_respects_every_capacity(shape, world, mbpr, hbm, dram, nvme):
    budget = planner.MemoryBudget(hbm * GiB, dram * GiB, nvme * GiB)
    split = planner.plan(shape, world, mbpr, budget, unit_buffers=3)
    if split is None:
        return
    shard = shape.num_layers * shape.layer_numel / world
    sizes = {"parameter": shard * 2.0, "optimizer": shard * 12.0,
             "checkpoint": shape.num_layers * mbpr * shape.tokens_per_micro_batch * shape.hidden * 2.0}
    used = {"hbm": 0.0, "dram": 0.0, "nvme": 0.0}
    for kind, total in sizes.items():
        g, c = split[kind]
        assert 0.0 <= g <= 1.0 and 0.0 <= c <= 1.0 and g + c <= 1.0 + 1e-9, (kind, split[kind])
        used["hbm"] += g * total
        used["dram"] += c * total
        used["nvme"] += (1.0 - g - c) * total
    ws = planner.working_set_bytes(shape, world, mbpr, 3, True, 1)
    slack = 0.002 * sum(sizes.values()) + 1.0          # ratios are rounded to 4 digits
    assert used["hbm"] + ws <= budget.hbm_bytes + slack
    assert used["dram"] <= budget.dram_bytes + slack
    assert used["nvme"] <= budget.nvme_bytes + slack
    assert split["gradient"] == [1.0, 0.0]


@settings(max_examples=60, deadline=None)
@given(shape=shapes, world=st.sampled_from([1, 2, 8]), hbm=st.floats(30, 120))
def test_more_hbm_never_moves_state_off_the_gpu(shape, world, hbm):
    def gpu_bytes(h):
        split = planner.plan(shape, world, 1, planner.MemoryBudget(h * GiB, 4000 * GiB, 0.0), unit_buffers=3)
        if split is None:
            return None
        shard = shape.num_layers * shape.layer_numel / world
        return split["parameter"][0] * shard * 2 + split["optimizer"][0] * shard * 12
    small, large = gpu_bytes(hbm), gpu_bytes(hbm + 40)
    if small is None:
        return
    assert large is not None and large >= small - 1e-3 * abs(small) - 1.0
