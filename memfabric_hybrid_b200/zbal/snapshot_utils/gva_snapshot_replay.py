"""Replays the allocation trace of a snapshot through the symmetric-heap allocator running over a made-up address range
(no device needed), and returns the snapshot of the replayed heap: does a recorded workload still fit, and how does it
lay out, after a change of the allocator's policy or settings (``ZBAL_ALLOC_CONF``)?
Parity: app/zbal/simulator/python/snapshot_utils/gva_snapshot_replay.py of the reference."""
from __future__ import annotations

import ctypes as C
from typing import Optional

DEFAULT_BASE = 0x100000000000


def replay_snapshot(snapshot: dict, device_id: int = 0, shmem_size: int = 62277025792, dump_replay_snapshot: bool = True,
                    base_addr: Optional[int] = None):
    """``snapshot``: the memory visualiser's layout (``device_traces[device_id]`` with alloc / free_completed /
    empty_cache entries). This REPLACES the allocator of the calling process by a simulated one of ``shmem_size`` bytes:
    run it offline. Returns the replayed heap in the same layout (None with ``dump_replay_snapshot=False``); its
    ``replay`` entry counts the events, the allocations that failed and those that landed at another offset."""
    from .. import _capi as K
    from .. import module as M
    trace = snapshot["device_traces"][device_id]
    first = next((te["addr"] for te in trace if te["action"] == "segment_alloc"), None)
    base = base_addr if base_addr is not None else (first if first is not None else DEFAULT_BASE)
    l = K.lib()
    l.zbal_sma_uninit(0)
    l.zbal_simulate_init(base, shmem_size)
    if dump_replay_snapshot:
        M.record_memory_history("all", 0xFFFFFFFF)
    live = {}
    events = failed = moved = 0
    for te in trace:
        action = te["action"]
        if action == "alloc":
            events += 1
            p = l.zbal_pluggable_malloc(te["size"], 0, C.c_void_p(te.get("stream", 0)))
            if not p:
                failed += 1
                continue
            if first is not None and p - base != te["addr"] - first:
                moved += 1
            live[te["addr"]] = p
        elif action == "free_completed":
            events += 1
            p = live.pop(te["addr"], None)
            if p:
                l.zbal_pluggable_free(p, 0, 0, None)
        elif action == "empty_cache":
            events += 1
            l.zbal_pluggable_empty_cache(False)
    if not dump_replay_snapshot:
        return None
    out = M.memviz_snapshot()
    M.record_memory_history(None, 0)
    out["replay"] = {"events": events, "failed": failed, "moved": moved, "live": len(live)}
    return out
