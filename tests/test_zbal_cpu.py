"""zbal host side without a GPU: the split heap and the caching allocator on a made-up address range, and
bootstrap / communicator bookkeeping over the fake device backend with real processes."""
import ctypes as C
import json
import os

import pytest

from conftest import free_port
from mp_util import run_ranks

BASE = 0x7000_0000_0000
MiB = 1 << 20


@pytest.fixture()
def sma():
    from memfabric_hybrid_b200.zbal import _capi as K
    l = K.lib()
    l.zbal_simulate_init(BASE, 256 * MiB)
    yield l
    l.zbal_sma_uninit(0)


def _stats(l):
    from memfabric_hybrid_b200.zbal import _capi as K
    s = K.SmaStatsC()
    assert l.zbal_sma_get_stats(C.byref(s)) == 0
    return s


def test_small_low_large_high_and_rounding(sma):
    a = sma.zbal_pluggable_malloc(1000, 0, None)
    b = sma.zbal_pluggable_malloc(100, 0, None)
    big = sma.zbal_pluggable_malloc(3 * MiB + 1, 0, None)
    assert a == BASE and b == BASE + 1024          # 1000 -> 1024, packed from the low end
    assert big == BASE + 256 * MiB - 4 * MiB       # rounded to 2 MiB steps, carved from the high end
    s = _stats(sma)
    assert s.inUseBytes == 1024 + 512 + 4 * MiB and s.heapCarves == 3 and s.cacheHits == 0
    for p in (a, b, big):
        sma.zbal_pluggable_free(p, 0, 0, None)
    assert _stats(sma).inUseBytes == 0 and _stats(sma).cachedBytes == 1024 + 512 + 4 * MiB


def test_allocator_configuration_keys(monkeypatch):
    """segment_size_mb (rounding granule of large requests) and small_heap_size (bytes of the low end that small requests
    may occupy; further small requests are carved from the high end) from ZBAL_ALLOC_CONF; unknown keys are ignored."""
    from memfabric_hybrid_b200.zbal import _capi as K
    monkeypatch.setenv("ZBAL_ALLOC_CONF", "segment_size_mb:8,small_heap_size:4096,small_heap_threshold:65536,use_sma_allocator:True,"
                                            "use_vmm_for_static_memory:False,bogus_key:1")
    l = K.lib()
    l.zbal_simulate_init(BASE, 256 * MiB)
    try:
        big = l.zbal_pluggable_malloc(3 * MiB, 0, None)
        assert big == BASE + 256 * MiB - 8 * MiB            # 3 MiB rounded to the 8 MiB segment granule
        smalls = [l.zbal_pluggable_malloc(1024, 0, None) for _ in range(5)]
        assert smalls[:4] == [BASE + i * 1024 for i in range(4)]     # 4096 bytes of small heap
        assert BASE + 4096 <= smalls[4] and smalls[4] >= BASE + 128 * MiB   # the fifth no longer fits below the limit: high end
        mid = l.zbal_pluggable_malloc(32768, 0, None)       # below the (lowered) threshold of 64 KiB: small, and too big for what is left
        assert mid >= BASE + 128 * MiB
        for p in smalls + [big, mid]:
            l.zbal_pluggable_free(p, 0, 0, None)
    finally:
        l.zbal_sma_uninit(0)


def test_cache_is_per_stream_and_flush_on_exhaustion(sma):
    s1, s2 = C.c_void_p(0x10), C.c_void_p(0x20)
    p = sma.zbal_pluggable_malloc(8 * MiB, 0, s1)
    sma.zbal_pluggable_free(p, 0, 0, s1)
    q = sma.zbal_pluggable_malloc(8 * MiB, 0, s2)   # another stream must not take the cached block
    assert q != p
    r = sma.zbal_pluggable_malloc(7 * MiB, 0, s1)   # same stream: a slightly smaller request reuses it
    assert r == p and _stats(sma).cacheHits == 1
    sma.zbal_pluggable_free(q, 0, 0, s2)
    sma.zbal_pluggable_free(r, 0, 0, s1)
    # 16 MiB sit in the caches; a request that only fits once they are returned must succeed
    huge = sma.zbal_pluggable_malloc(250 * MiB, 0, s1)
    assert huge != 0 and _stats(sma).cachedBytes == 0
    assert sma.zbal_pluggable_malloc(64 * MiB, 0, s1) is None and _stats(sma).failedMallocs == 1
    from memfabric_hybrid_b200.zbal import _capi as K
    assert "exhausted" in K.last_error()
    sma.zbal_pluggable_free(huge, 0, 0, s1)
    sma.zbal_pluggable_empty_cache(True)
    assert _stats(sma).largestFreeBlock == 256 * MiB   # everything coalesced back into one block


def test_private_pool_keeps_graph_blocks_apart(sma):
    """Capture-style pools: tagged blocks are parked in their pool when freed, survive empty_cache, are reused only
    by the same pool, and return to the heap when the pool is released."""
    cap, other = C.c_void_p(0x10), C.c_void_p(0x20)
    FILTER = C.CFUNCTYPE(C.c_bool, C.c_void_p, C.c_void_p)
    only_cap = FILTER(lambda ctx, stream: stream == cap.value)
    pool = (0, 7)
    assert sma.zbal_sma_begin_pool(*pool, C.cast(only_cap, C.c_void_p), None) == 0
    a = sma.zbal_pluggable_malloc(4 * MiB, 0, cap)       # tagged
    b = sma.zbal_pluggable_malloc(4 * MiB, 0, other)     # the filter rejects this stream: ordinary block
    sma.zbal_pluggable_free(a, 0, 0, cap)
    s = _stats(sma)
    assert s.poolCount == 1 and s.poolCachedBytes == 4 * MiB and s.cachedBytes == 0
    a2 = sma.zbal_pluggable_malloc(4 * MiB, 0, cap)      # the same pool reuses its parked block
    assert a2 == a
    assert sma.zbal_sma_end_pool(*pool) == 0             # capture over: the graph now owns a2's address
    sma.zbal_pluggable_free(a2, 0, 0, cap)
    sma.zbal_pluggable_free(b, 0, 0, other)
    sma.zbal_pluggable_empty_cache(True)                 # returns b, must leave the pool alone
    assert _stats(sma).poolCachedBytes == 4 * MiB and _stats(sma).cachedBytes == 0
    got = [sma.zbal_pluggable_malloc(4 * MiB, 0, cap) for _ in range(8)]
    assert a not in got                                  # nobody else gets the graph's block
    for p in got:
        sma.zbal_pluggable_free(p, 0, 0, cap)
    assert sma.zbal_sma_begin_pool(*pool, None, None) == 0    # a second capture into the same pool (NULL filter: all streams)
    assert sma.zbal_pluggable_malloc(4 * MiB, 0, other) == a
    sma.zbal_pluggable_free(a, 0, 0, other)
    assert sma.zbal_sma_end_pool(*pool) == 0
    assert sma.zbal_sma_release_pool(*pool) == 0 and sma.zbal_sma_release_pool(*pool) != 0
    sma.zbal_pluggable_empty_cache(True)
    s = _stats(sma)
    assert s.poolCount == 0 and s.poolCachedBytes == 0 and s.largestFreeBlock == 256 * MiB


def test_same_sequence_gives_same_offsets_and_snapshot(sma):
    import random
    from memfabric_hybrid_b200.zbal import module as M

    def run(seed):
        rnd = random.Random(seed)
        live, trace = [], []
        for _ in range(400):
            if live and rnd.random() < 0.45:
                sma.zbal_pluggable_free(live.pop(rnd.randrange(len(live))), 0, 0, None)
            else:
                size = rnd.choice([64, 700, 4096, 100_000, 3 * MiB, 9 * MiB])
                p = sma.zbal_pluggable_malloc(size, 0, None)
                assert p
                live.append(p)
                trace.append(p - BASE)
        for p in live:
            sma.zbal_pluggable_free(p, 0, 0, None)
        sma.zbal_pluggable_empty_cache(True)
        return trace

    sma.zbal_sma_record_history(True, 100)
    first = run(3)
    snap = M.snapshot()
    assert snap["heap"]["size"] == 256 * MiB and snap["heap"]["in_use"] == 0
    assert len(snap["history"]) == 100 and snap["history"][-1]["op"] == "empty_cache"
    assert [b["state"] for b in snap["blocks"]] == ["free"]
    assert run(3) == first                       # determinism is what makes the heap symmetric across ranks
    json.dumps(snap)


def test_replay_tool_reports_fragmentation(tmp_path, sma):
    from memfabric_hybrid_b200.zbal import module as M, simulator
    sma.zbal_sma_record_history(True, 0)
    ps = [sma.zbal_pluggable_malloc(3 * MiB, 0, None) for _ in range(8)]
    for p in ps[::2]:
        sma.zbal_pluggable_free(p, 0, 0, None)
    path = tmp_path / "snap.json"
    M.dump_snapshot(str(path))
    rep = simulator.analyse(json.loads(path.read_text()))
    assert rep["active_bytes"] == 4 * 4 * MiB and rep["cached_bytes"] == 4 * 4 * MiB and rep["blocks"] >= 9
    # replaying the recorded history on a fresh heap reproduces the addresses
    out = simulator.replay(json.loads(path.read_text()))
    assert out["mismatches"] == 0 and out["events"] == 12
    txt = simulator.render(json.loads(path.read_text()), width=64)
    assert "#" in txt and "." in txt


def test_visualiser_layout_snapshot_model_replay_and_exports(tmp_path, sma):
    """zbal.dump_snapshot() in the memory visualiser's layout, the address-ordered model built from its trace, a replay
    through the allocator, the drawings and the Chrome-trace export (names of the reference's snapshot_utils)."""
    import pickle

    import zbal
    from snapshot_utils.gva_layout_analyzer import Block, MemoryAllocatorSimulator
    from snapshot_utils.gva_layout_viz import (parse_mem_to_profile, parser_file_ops, visualize_file_memory, visualize_file_snapshot,
                                               visualize_sim_memory)
    from snapshot_utils.gva_snapshot_replay import replay_snapshot
    zbal.record_memory_history("all", 1 << 40)          # the reference's spelling; an over-long limit is clamped
    ps = [sma.zbal_pluggable_malloc(3 * MiB, 0, None) for _ in range(6)]
    small = sma.zbal_pluggable_malloc(4096, 0, None)
    for p in ps[1::2]:
        sma.zbal_pluggable_free(p, 0, 0, None)
    sma.zbal_pluggable_empty_cache(False)
    snap = zbal.dump_snapshot()
    assert set(snap) == {"segments", "device_traces"} and len(snap["segments"]) == 1
    seg = snap["segments"][0]
    assert seg["address"] == BASE and seg["total_size"] == 256 * MiB and seg["allocated_size"] == 3 * 4 * MiB + 4096
    assert sum(b["size"] for b in seg["blocks"]) == 256 * MiB                        # the blocks tile the segment
    assert [b["address"] for b in seg["blocks"]] == sorted(b["address"] for b in seg["blocks"])
    assert sum(1 for b in seg["blocks"] if b["state"] == "active_allocated") == 4
    trace = snap["device_traces"][0]
    acts = [te["action"] for te in trace]
    assert acts[0] == "segment_alloc" and acts.count("alloc") == 7 and acts.count("free_completed") == 3 and "empty_cache" in acts

    # the model of the trace agrees with the snapshot's block list
    sim = MemoryAllocatorSimulator(gva_size=256 * MiB).simulate(trace)
    assert sim.gva_base_addr == BASE and sim.get_all_segments() == [(BASE, BASE + 256 * MiB)]
    used = sim.get_used_blocks()
    assert {(b.addr, b.size) for b in used} == {(b["address"], b["size"]) for b in seg["blocks"] if b["state"] == "active_allocated"}
    assert sum(b.size for b in sim.get_all_blocks()) == 256 * MiB and sim.used_bytes() == seg["allocated_size"]
    assert all(isinstance(b, Block) and b.status == "FREE" for b in sim.get_free_blocks()) and 0.0 <= sim.fragmentation() < 1.0
    assert sim.get_free_space() == [0]                                                # one segment covers the whole range
    # misuse is refused
    with pytest.raises(ValueError):
        sim._alloc(used[0].addr, 512)
    with pytest.raises(ValueError):
        sim._free(BASE + 12345)
    with pytest.raises(ValueError):
        sim._segment_free(BASE)                                                       # still has blocks in use
    # holes between segments
    two = MemoryAllocatorSimulator(gva_base_addr=0, gva_size=100)
    two.simulate([{"action": "segment_alloc", "addr": 10, "size": 20}, {"action": "segment_alloc", "addr": 50, "size": 10},
                  {"action": "alloc", "addr": 12, "size": 4}, {"action": "alloc", "addr": 16, "size": 4}, {"action": "free_completed", "addr": 12},
                  {"action": "free_completed", "addr": 16}])
    assert two.get_free_space() == [10, 20, 40] and [(b.addr, b.size) for b in two.get_all_blocks()] == [(10, 20), (50, 10)]
    two.simulate([{"action": "segment_free", "addr": 50, "size": 10}])
    assert two.get_free_space() == [10, 70]

    # files: pickle in the visualiser's layout, JSON in the allocator's own; both load as a trace
    zbal.dump_snapshot(str(tmp_path / "s.pkl"))
    zbal.dump_snapshot(str(tmp_path / "s.json"))
    assert pickle.loads((tmp_path / "s.pkl").read_bytes())["segments"][0]["address"] == BASE
    assert [te["action"] for te in parser_file_ops(str(tmp_path / "s.pkl"))] == acts
    assert [te["action"] for te in parser_file_ops(str(tmp_path / "s.json"))] == acts
    assert parser_file_ops(str(tmp_path / "s.pkl"), get_traces=False)[0]["total_size"] == 256 * MiB
    with pytest.raises(ValueError):
        parser_file_ops(str(tmp_path / "s.txt"))

    # drawings
    svg = visualize_sim_memory(sim, display_segments=True, output=str(tmp_path / "sim.svg"))
    assert svg.startswith("<svg") and svg.count("<rect") >= 1 + 1 + 4 and (tmp_path / "sim.svg").read_text() == svg
    svg2 = visualize_file_memory(0.25, hex(BASE), trace)
    assert svg2.count(_used_colour()) >= 4
    gaps = visualize_file_snapshot(0, BASE, [{"address": 0, "total_size": 10, "blocks": []}, {"address": 30, "total_size": 10, "blocks": []},
                                             {"address": 45, "total_size": 5, "blocks": [{"address": 45, "size": 5, "state": "inactive"}]}],
                                   output=str(tmp_path / "gaps.svg"))
    assert [(g["gap_start"], g["size"]) for g in gaps] == [(10, 20), (40, 5)] and (tmp_path / "gaps.svg").exists()
    assert visualize_file_snapshot(0.25, BASE, snap["segments"]) == []

    # Chrome trace: 3 lifetimes that ended, 4 still alive
    n = parse_mem_to_profile(trace, str(tmp_path / "prof.json"), export_segments=False, with_unfree=True)
    ev = json.loads((tmp_path / "prof.json").read_text())["traceEvents"]
    assert len(ev) == n and sum(1 for e in ev if e["ph"] == "X" and e["name"].startswith("Block_")) == 3
    assert sum(1 for e in ev if e["name"].startswith("Unfreed_")) == 4 and {e["tid"] for e in ev if e["ph"] == "X"} == {"< 16MB (Small)"}
    assert [e["args"]["Allocated_MB"] for e in ev if e["ph"] == "C"][-1] == pytest.approx((3 * 4 * MiB + 4096) / MiB)
    parse_mem_to_profile(trace, str(tmp_path / "seg.json"))
    assert sum(1 for e in json.loads((tmp_path / "seg.json").read_text())["traceEvents"] if e["ph"] == "C") == 1

    # replay through the allocator on another base: the same layout, shifted
    out = replay_snapshot(snap, shmem_size=256 * MiB, base_addr=BASE + (1 << 40))
    assert out["replay"] == {"events": 11, "failed": 0, "moved": 0, "live": 4}
    again = MemoryAllocatorSimulator(gva_size=256 * MiB).simulate(out["device_traces"][0])
    assert again == sim and again.gva_base_addr == BASE + (1 << 40)
    assert not (again == MemoryAllocatorSimulator(gva_size=256 * MiB).simulate(trace[:5]))
    del small


def _used_colour():
    from memfabric_hybrid_b200.zbal.snapshot_utils.gva_layout_viz import _COL
    return _COL["used"]


def _boot(rank, world, port):
    os.environ["MF_DEVICE_BACKEND"] = "fake"
    import memfabric_hybrid_b200.zbal as z
    from memfabric_hybrid_b200.zbal import _capi as K
    l = K.lib()
    assert not z.is_initialized()
    assert z.zbal_init(world, 0, rank, 256 << 20, ip_port=f"127.0.0.1:{port}", start_config_server=True, comm_group_cap=4)
    with pytest.raises(K.ZbalError):
        z.zbal_init(world, 0, rank, 256 << 20, ip_port=f"127.0.0.1:{port}")
    out = z.module.bootstrap_output()
    assert out.localGva == out.baseGva + rank * out.symmetricSize and out.heapGva == out.localGva + out.commAreaSize
    p = K.CommPropertyC()
    g = l.zbal_comm_get_global()
    assert l.zbal_comm_get_property(g, C.byref(p)) == 0
    assert (p.name, p.groupId, p.groupSize, p.groupRank) == (b"zbal_world", 0, world, rank)
    # two strided sub-groups created at the same time agree on different slots
    first = rank % 2
    o = K.CommOptionsC()
    o.name, o.firstRank, o.rankStep, o.groupSize = f"zbal_{first}:{first + 2}:2_group_0".encode(), first, 2, 2
    h = C.c_void_p()
    assert l.zbal_comm_create(C.byref(o), C.byref(h)) == 0
    assert l.zbal_comm_get_property(h, C.byref(p)) == 0
    slot, grank = p.groupId, p.groupRank
    assert grank == rank // 2 and 1 <= slot <= 3 and l.zbal_comm_get_by_name(o.name) == h.value
    # not a member / duplicate name / leaves the world
    bad = K.CommOptionsC()
    bad.name, bad.firstRank, bad.rankStep, bad.groupSize = b"x", 1 - first, 2, 2
    assert l.zbal_comm_create(C.byref(bad), C.byref(C.c_void_p())) != 0
    assert l.zbal_comm_create(C.byref(o), C.byref(C.c_void_p())) != 0
    bad.firstRank, bad.groupSize = first, 3
    assert l.zbal_comm_create(C.byref(bad), C.byref(C.c_void_p())) != 0
    # allocations land at the same offset of every rank's heap
    a = l.zbal_pluggable_malloc(5000, 0, None) - out.heapGva
    assert l.zbal_comm_destroy(h, 0) == 0 and l.zbal_comm_get_by_name(o.name) is None
    assert z.zbal_uninit() and not z.is_initialized()
    return slot, a


def test_bootstrap_and_communicators_over_fake_backend():
    res = run_ranks(_boot, 4, (free_port(),), timeout=120)
    slots = [r[0] for r in res]
    assert slots[0] == slots[2] and slots[1] == slots[3] and slots[0] != slots[1]
    assert len({r[1] for r in res}) == 1


def test_balance_matrix_plan():
    """The helper plan: nothing to do below the threshold; an overloaded rank's overflow goes to ranks with room."""
    import numpy as np
    from memfabric_hybrid_b200.zbal import _capi as K
    l = K.lib()
    f = l.zbal_moe_balance_matrix
    f.restype = C.c_int32
    f.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_float, C.c_float, C.c_uint32, C.c_void_p]
    ranks, experts, topk = 4, 8, 2

    def plan(tokens, min_tokens=128):
        counts = np.zeros((ranks, experts), dtype=np.int32)
        for r, t in enumerate(tokens):
            counts[r, 0] = t * topk
        m = np.empty((ranks, ranks * 2), dtype=np.int32)
        assert f(counts.ctypes.data, ranks, experts, topk, 1.2, 1.0, min_tokens, m.ctypes.data) == 0
        return m.reshape(ranks, ranks, 2)
    small = plan([100, 50, 10, 0])
    for r, t in enumerate([100, 50, 10, 0]):
        assert tuple(small[r, r]) == ((0, t) if t else (-1, -1))
    assert (small[~np.eye(ranks, dtype=bool)] == -1).all()
    big = plan([4000, 400, 400, 400])                       # avg 1300: rank 0 may keep 1560, others may hold 1300
    assert tuple(big[0, 0]) == (0, 1560)
    covered = sorted(tuple(big[h, 0]) for h in range(ranks) if big[h, 0, 0] >= 0)
    assert covered[0][0] == 0 and covered[-1][1] == 4000 and all(covered[i][1] == covered[i + 1][0] for i in range(len(covered) - 1))
    load = [sum(int(big[h, o, 1] - big[h, o, 0]) for o in range(ranks) if big[h, o, 0] >= 0) for h in range(ranks)]
    assert load[0] == 1560 and max(load[1:]) <= 1300 and sum(load) == 5200


def _native_pg(rank, world, port):
    """The C++ c10d backend over the fake device backend: routing, naming and fall-backs, no GPU needed."""
    os.environ.update(MF_DEVICE_BACKEND="fake", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch
    import torch.distributed as dist
    import memfabric_hybrid_b200.zbal as z
    from memfabric_hybrid_b200.zbal import process_group as P
    assert P.implementation() == "native", "lib/_zbal_c10d.so is not built"
    assert z.zbal_init(world, 0, rank, 256 << 20, ip_port=f"127.0.0.1:{port + 7}", start_config_server=True, comm_group_cap=8)
    dist.init_process_group("zbal", rank=rank, world_size=world, init_method=f"tcp://127.0.0.1:{port}")
    be = dist.group.WORLD._get_backend(torch.device("cpu"))
    assert type(be).__name__ == "ProcessGroupZBAL" and type(be).__module__ == "_zbal_c10d"
    assert be.strided and be.comm_name() == "zbal_world" and dist.get_backend() == "zbal"
    t = torch.full((4,), rank + 1.0)
    dist.all_reduce(t)                                   # host tensor: the gloo fall-back built through the factory
    assert t.tolist() == [float(sum(range(1, world + 1)))] * 4
    objs = [None] * world
    dist.all_gather_object(objs, {"r": rank})
    assert [o["r"] for o in objs] == list(range(world))
    dist.barrier()
    names = []
    for ranks in ([0, 2], [1, 3], [0, 1, 3]):
        g = dist.new_group(ranks)
        if rank in ranks:
            b = g._get_backend(torch.device("cpu"))
            names.append(b.comm_name() if b.strided else "irregular")
            x = torch.tensor([float(rank)])
            dist.all_reduce(x, group=g)
            assert x.item() == float(sum(ranks))
    dist.barrier()
    dist.destroy_process_group()
    assert z.zbal_uninit()
    return names


def test_native_c10d_backend_routing_and_group_names():
    res = run_ranks(_native_pg, 4, (free_port(),), timeout=180)
    assert res[0] == ["zbal_0:2:2_group_0", "irregular"] and res[2] == ["zbal_0:2:2_group_0"]
    assert res[1] == ["zbal_1:3:2_group_0", "irregular"] and res[3] == ["zbal_1:3:2_group_0", "irregular"]


def test_heap_grows_by_segments(monkeypatch):
    """Expandable segments on the simulated heap: a second address range is added by hand, and by the grow hook when a
    request no longer fits (ZBAL_ALLOC_CONF=expandable_segments:True)."""
    from memfabric_hybrid_b200.zbal import _capi as K
    l = K.lib()
    HOOK = C.CFUNCTYPE(C.c_int, C.c_uint64, C.c_void_p)
    l.zbal_sma_set_grow_hook.argtypes = [HOOK, C.c_void_p]
    l.zbal_sma_set_grow_hook.restype = None
    calls = []

    def grow(need, _ctx):
        calls.append(need)
        if len(calls) > 2:
            return -1
        return l.zbal_sma_add_segment(BASE + (1 << 32) * len(calls), 64 * MiB)

    cb = HOOK(grow)
    try:
        # off: exhaustion is an error, a segment can still be added by hand
        monkeypatch.setenv("ZBAL_ALLOC_CONF", "expandable_segments:False")
        l.zbal_simulate_init(BASE, 64 * MiB)
        l.zbal_sma_set_grow_hook(cb, None)
        a = l.zbal_pluggable_malloc(48 * MiB, 0, None)
        assert a and not l.zbal_pluggable_malloc(32 * MiB, 0, None) and calls == []
        assert l.zbal_sma_add_segment(BASE + (1 << 40), 64 * MiB) == 0
        assert l.zbal_sma_add_segment(BASE + (1 << 40) + MiB, 4 * MiB) != 0          # overlaps
        b = l.zbal_pluggable_malloc(32 * MiB, 0, None)
        assert BASE + (1 << 40) <= b < BASE + (1 << 40) + 64 * MiB
        s = _stats(l)
        assert s.segments == 2 and s.segmentsAdded == 0 and s.heapSize == 128 * MiB
        l.zbal_sma_uninit(0)
        # on: the hook is asked, at most max_segments - 1 times
        monkeypatch.setenv("ZBAL_ALLOC_CONF", "expandable_segments:True,max_segments:3")
        l.zbal_simulate_init(BASE, 64 * MiB)
        got = [l.zbal_pluggable_malloc(40 * MiB, 0, None) for _ in range(4)]
        assert all(got[:3]) and not got[3]
        assert got[1] >= BASE + (1 << 32) and got[2] >= BASE + (2 << 32) and len(calls) == 2
        s = _stats(l)
        assert s.segments == 3 and s.segmentsAdded == 2 and s.failedMallocs == 1
        # released memory of a segment is reused like any other
        l.zbal_pluggable_free(got[1], 40 * MiB, 0, None)
        l.zbal_pluggable_empty_cache(False)
        assert l.zbal_pluggable_malloc(40 * MiB, 0, None) == got[1]
    finally:
        l.zbal_sma_set_grow_hook(HOOK(0), None)
        l.zbal_sma_uninit(0)


def _boot_expand(rank, world, port):
    os.environ["MF_DEVICE_BACKEND"] = "fake"
    os.environ["ZBAL_ALLOC_CONF"] = "expandable_segments:True,max_segments:3"
    import memfabric_hybrid_b200.zbal as z
    from memfabric_hybrid_b200.zbal import _capi as K
    l = K.lib()
    assert z.zbal_init(world, 0, rank, 64 << 20, ip_port=f"127.0.0.1:{port}", start_config_server=True, comm_group_cap=2)
    out = z.module.bootstrap_output()
    # explicit, collective
    base, size = z.expand_heap()
    assert size == 64 << 20
    delta = base - out.localGva
    # automatic: the same request sequence on every rank runs out of room at the same call
    blocks = [l.zbal_pluggable_malloc(30 << 20, 0, None) for _ in range(5)]
    assert all(blocks), blocks
    st = z.heap_stats()
    z.zbal_uninit()
    return delta, [b - out.localGva for b in blocks], st["segments"], st["segmentsAdded"]


def test_symmetric_heap_expands_collectively_over_fake_backend():
    res = run_ranks(_boot_expand, 2, (free_port(),), timeout=120)
    assert res[0] == res[1]                      # same distance to the new segment, same offsets of every block
    assert res[0][2] == 3 and res[0][3] == 1     # one segment by hand, one by the hook
