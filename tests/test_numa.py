"""NUMA placement logic against a fake sysfs tree (no GPU, no real topology needed)."""
import os

from flextrain_b200.utils import numa


def _fake_sysfs(root, gpu_nodes, node_lists):
    for i, node in enumerate(gpu_nodes):
        d = root / "bus/pci/devices" / numa.pci_address(0, 0x10 + i, 0)
        d.mkdir(parents=True)
        (d / "numa_node").write_text(f"{node}\n")
    for node, text in node_lists.items():
        d = root / f"devices/system/node/node{node}"
        d.mkdir(parents=True)
        (d / "cpulist").write_text(text + "\n")
    return str(root)


def test_cpulist_forms():
    assert numa.parse_cpulist("0-3,8,10-11\n") == [0, 1, 2, 3, 8, 10, 11]
    assert numa.parse_cpulist("5") == [5]
    assert numa.parse_cpulist("") == []


def test_eight_gpus_on_two_sockets_split_their_nodes_evenly(tmp_path):
    sysfs = _fake_sysfs(tmp_path, [0, 0, 0, 0, 1, 1, 1, 1], {0: "0-15,32-47", 1: "16-31,48-63"})
    nodes = [numa.gpu_numa_node(numa.pci_address(0, 0x10 + i, 0), sysfs) for i in range(8)]
    assert nodes == [0, 0, 0, 0, 1, 1, 1, 1]
    allowed = range(64)
    plans = [numa.plan_affinity(r, nodes, allowed, sysfs) for r in range(8)]
    assert all(len(p) == 8 for p in plans)
    flat = [c for p in plans for c in p]
    assert sorted(flat) == list(range(64))                       # every CPU used once
    assert set(plans[0]) <= set(numa.node_cpus(0, sysfs)) and set(plans[5]) <= set(numa.node_cpus(1, sysfs))


def test_cpuset_restrictions_and_unknown_topology(tmp_path):
    sysfs = _fake_sysfs(tmp_path, [0, -1], {0: "0-7"})
    nodes = [0, -1]
    assert numa.plan_affinity(0, nodes, {2, 3, 9}, sysfs) == [2, 3]     # only what the cpuset allows
    assert numa.plan_affinity(1, nodes, range(8), sysfs) is None         # the platform does not say
    assert numa.plan_affinity(0, nodes, {20, 21}, sysfs) is None         # node outside the cpuset
    assert numa.plan_affinity(0, [3], range(8), sysfs) is None           # node without a cpulist
    assert numa.gpu_numa_node("0000:ff:00.0", sysfs) == -1


def test_binding_applies_and_failures_leave_the_process_alone(tmp_path):
    before = os.sched_getaffinity(0)
    omp = os.environ.get("OMP_NUM_THREADS")
    try:
        some = sorted(before)[: max(1, len(before) // 2)]
        sysfs = _fake_sysfs(tmp_path, [0], {0: ",".join(str(c) for c in some)})
        got = numa.bind_to_gpu_node(0, 1, sysfs, gpu_nodes=[0])
        assert got == some and os.sched_getaffinity(0) == set(some)
        # nothing known about the GPU: unchanged
        assert numa.bind_to_gpu_node(0, 1, sysfs, gpu_nodes=[-1]) is None
        assert os.sched_getaffinity(0) == set(some)
    finally:
        os.sched_setaffinity(0, before)
        if omp is None:
            os.environ.pop("OMP_NUM_THREADS", None)
        else:
            os.environ["OMP_NUM_THREADS"] = omp
        import torch
        torch.set_num_threads(max(1, len(before)))
