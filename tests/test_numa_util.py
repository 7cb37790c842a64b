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


def test_mem_scan_reads_free_memory_huge_pages_and_fragmentation(tmp_path, capsys):
    from memfabric_hybrid_b200.utils import mem_scan
    for n, (total, free) in enumerate([(64 << 20, 20 << 20), (64 << 20, 1 << 20)]):     # kB
        d = tmp_path / f"sys/devices/system/node/node{n}"
        (d / "hugepages/hugepages-2048kB").mkdir(parents=True)
        (d / "hugepages/hugepages-1048576kB").mkdir(parents=True)
        (d / "meminfo").write_text(f"Node {n} MemTotal:       {total} kB\nNode {n} MemFree:        {free} kB\nNode {n} HugePages_Total:     8\n")
        (d / "hugepages/hugepages-2048kB/nr_hugepages").write_text("8\n")
        (d / "hugepages/hugepages-2048kB/free_hugepages").write_text(f"{8 - 3 * n}\n")
        (d / "hugepages/hugepages-1048576kB/nr_hugepages").write_text("0\n")
        (d / "hugepages/hugepages-1048576kB/free_hugepages").write_text("0\n")
    (tmp_path / "proc").mkdir()
    # node 0: DMA32 + Normal zones; node 1: only small blocks (fragmented)
    (tmp_path / "proc/buddyinfo").write_text(
        "Node 0, zone    DMA32      1      0      0      0      0      0      0      0      0      1      2\n"
        "Node 0, zone   Normal    100     50      0      0      0      0      0      0      0      3      5\n"
        "Node 1, zone   Normal   4000   2000    100      0      0      0      0      0      0      0      0\n")
    rep = mem_scan.scan(2 << 20, str(tmp_path), page=4096)
    n0, n1 = rep["nodes"]
    assert n0["total_bytes"] == 64 << 30 and n0["free_bytes"] == 20 << 30 and n1["free_bytes"] == 1 << 30
    assert n0["hugepages"]["2048kB"] == {"total": 8, "free": 8} and n1["hugepages"]["2048kB"]["free"] == 5
    assert n0["largest_free_run_bytes"] == 4096 << 10 and n1["largest_free_run_bytes"] == 4096 << 2
    assert n0["free_in_runs_of_min_bytes"] == 4 * (4096 << 9) + 7 * (4096 << 10)      # orders 9 and 10 only
    assert n1["free_in_runs_of_min_bytes"] == 0
    assert n0["free_in_buddy_bytes"] == n0["free_in_runs_of_min_bytes"] + 101 * 4096 + 50 * 8192
    assert rep["total_free_bytes"] == 21 << 30 and rep["total_free_in_runs_of_min_bytes"] == n0["free_in_runs_of_min_bytes"]
    assert mem_scan.main(["--root", str(tmp_path)]) == 0
    out = capsys.readouterr().out
    assert "node" in out and "2048kB: 5/8" in out
    # a container that shows nothing
    empty = mem_scan.scan(root=str(tmp_path / "nowhere"))
    assert empty["nodes"] == [] and empty["total_free_bytes"] is None and "no NUMA information" in mem_scan.render(empty)
    assert mem_scan.main(["--json"]) == 0                                           # this machine, whatever it shows
