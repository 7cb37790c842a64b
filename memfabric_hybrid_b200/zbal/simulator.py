"""Offline tools for allocator snapshots (``zbal.dump_snapshot``): layout analysis, a text map of the heap,
and a replay of the recorded malloc/free history on a simulated heap to see whether a sequence still
fits after a change of policy or settings.

    python -m memfabric_hybrid_b200.zbal.simulator snapshot.json [--replay] [--width 100]

Parity of role: app/zbal/simulator/python of the reference (snapshot replay, layout analyser, visualiser).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json


def analyse(snap: dict) -> dict:
    """Totals and fragmentation of a snapshot's block list."""
    blocks = snap["blocks"]
    by = {"active": 0, "cached": 0, "free": 0}
    largest_free = 0
    for b in blocks:
        by[b["state"]] += b["size"]
        if b["state"] == "free":
            largest_free = max(largest_free, b["size"])
    thr = snap["heap"]["threshold"]
    small = sum(1 for b in blocks if b["state"] != "free" and b["size"] < thr)
    streams = sorted({b["stream"] for b in blocks if b["state"] == "active"})
    return {"heap_bytes": snap["heap"]["size"], "active_bytes": by["active"], "cached_bytes": by["cached"], "free_bytes": by["free"],
            "blocks": len(blocks), "small_blocks": small, "largest_free": largest_free,
            "fragmentation": 0.0 if by["free"] == 0 else 1.0 - largest_free / by["free"], "streams": streams,
            "history_events": len(snap.get("history", []))}


def render(snap: dict, width: int = 100) -> str:
    """One line per 1/16 of the heap; '#' in use, '+' cached, '.' free (the state covering most of each cell)."""
    base, size = snap["heap"]["base"], snap["heap"]["size"]
    cells = width * 16
    per = size / cells
    weight = [[0.0, 0.0, 0.0] for _ in range(cells)]
    col = {"active": 0, "cached": 1, "free": 2}
    for b in snap["blocks"]:
        lo, hi = b["addr"] - base, b["addr"] - base + b["size"]
        c0, c1 = int(lo / per), min(cells - 1, int((hi - 1) / per))
        for c in range(c0, c1 + 1):
            ov = min(hi, (c + 1) * per) - max(lo, c * per)
            if ov > 0:
                weight[c][col[b["state"]]] += ov
    chars = "".join("#+."[max(range(3), key=lambda k: w[k])] for w in weight)
    lines = [f"{int(i * size / 16) >> 20:>8} MiB |{chars[i * width:(i + 1) * width]}|" for i in range(16)]
    return "\n".join(lines)


def replay(snap: dict) -> dict:
    """Runs the recorded history on a fresh simulated heap of the same base and size. This REPLACES the
    allocator of the calling process: use it offline. Returns the number of events and how many mallocs
    landed at a different address than recorded (0 = the policy reproduced the layout)."""
    from . import _capi as K
    l = K.lib()
    l.zbal_sma_uninit(0)
    l.zbal_simulate_init(snap["heap"]["base"], snap["heap"]["size"])
    mismatches = failed = events = 0
    moved = {}
    for ev in snap.get("history", []):
        op = ev["op"]
        events += 1
        if op in ("malloc_heap", "malloc_cache"):
            p = l.zbal_pluggable_malloc(ev["requested"], 0, C.c_void_p(ev["stream"]))
            if not p:
                failed += 1
            elif p != ev["addr"]:
                mismatches += 1
            moved[ev["addr"]] = p
        elif op in ("free_cache", "free_heap"):
            p = moved.pop(ev["addr"], None)
            if p:
                l.zbal_pluggable_free(p, 0, 0, None)
        elif op == "empty_cache":
            l.zbal_pluggable_empty_cache(False)
    st = K.SmaStatsC()
    l.zbal_sma_get_stats(C.byref(st))
    return {"events": events, "mismatches": mismatches, "failed": failed, "peak_in_use": int(st.peakInUseBytes),
            "in_use": int(st.inUseBytes), "cached": int(st.cachedBytes)}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("snapshot")
    ap.add_argument("--replay", action="store_true")
    ap.add_argument("--width", type=int, default=100)
    a = ap.parse_args(argv)
    with open(a.snapshot) as f:
        snap = json.load(f)
    print(json.dumps(analyse(snap), indent=2))
    print(render(snap, a.width))
    if a.replay:
        print(json.dumps(replay(snap), indent=2))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
