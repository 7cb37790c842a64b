"""NUMA placement helper: sysfs parsing against a made-up tree; binding is a no-op where the information is missing."""
import os

from memfabric_hybrid_b200.utils import numa


def test_parse_cpulist():
    assert numa.parse_cpulist("0-3,8,10-11") == {0, 1, 2, 3, 8, 10, 11}
    assert numa.parse_cpulist("") == set() and numa.parse_cpulist("5") == {5}


def test_node_lookup_from_a_fake_sysfs(tmp_path, monkeypatch):
    dev = tmp_path / "bus/pci/devices/0000:1b:00.0"
    dev.mkdir(parents=True)
    (dev / "numa_node").write_text("1\n")
    node = tmp_path / "devices/system/node/node1"
    node.mkdir(parents=True)
    mine = sorted(os.sched_getaffinity(0))
    (node / "cpulist").write_text(f"{mine[0]}\n")
    monkeypatch.setattr(numa, "gpu_pci_address", lambda i: "0000:1b:00.0")
    assert numa.gpu_numa_node(0, str(tmp_path)) == 1 and numa.node_cpus(1, str(tmp_path)) == {mine[0]}
    before = os.sched_getaffinity(0)
    try:
        monkeypatch.setattr(numa, "prefer_node", lambda n: False)   # the made-up node does not exist on this host
        got = numa.bind_to_gpu(0, str(tmp_path))
        assert got["node"] == 1 and got["cpus"] == 1 and os.sched_getaffinity(0) == {mine[0]}
    finally:
        os.sched_setaffinity(0, before)
    # unknown node (-1) or no sysfs entry: nothing changes
    (dev / "numa_node").write_text("-1\n")
    assert numa.bind_to_gpu(0, str(tmp_path))["node"] is None and os.sched_getaffinity(0) == before
    monkeypatch.setattr(numa, "gpu_pci_address", lambda i: None)
    assert numa.bind_to_gpu(0, str(tmp_path))["node"] is None
