#!/usr/bin/env python
"""Host DRAM pool benchmark (the CPU-only configuration: 2 processes on one box, 64 MiB of pooled DRAM each, copies of
4 KiB - 8 MiB between a private host buffer and the PEER's slice of the pool, every transfer checked by CRC32).

The same script drives either implementation of the ``memfabric_hybrid`` Python API:

    python baseline/host_pool_cfg1.py --impl ours         # this repository's module
    python baseline/host_pool_cfg1.py --impl reference    # the unmodified reference, built with -DXPU_TYPE=NONE and
                                                          # laid out under baseline/_ref/memfabric_hybrid

It imports nothing but numpy and the chosen ``memfabric_hybrid``; what it measures is the public call
``BigMemory.copy_data`` (= ``smem_bm_copy``): local host -> global host (H2G, "LH2GH") into the peer's slice and global
host -> local host (G2H, "GH2LH") out of it, wall clock around a loop of synchronous calls, as the reference's own
bandwidth tool does (benchmark/bm/band_width_calculator.cpp:505-600). Prints one JSON line.
"""
import argparse
import json
import multiprocessing as mp
import os
import socket
import sys
import time
import zlib

HERE = os.path.dirname(os.path.abspath(__file__))
MIB = 1 << 20
SIZES = [4 << 10, 16 << 10, 64 << 10, 256 << 10, 1 << 20, 4 << 20, 8 << 20]


def _use(impl: str) -> None:
    root = os.path.dirname(HERE)
    sys.path[:] = [p for p in sys.path if os.path.abspath(p or ".") not in (root, HERE)]
    sys.path.insert(0, os.path.join(HERE, "_ref") if impl == "reference" else root)


def _rank(rank: int, impl: str, url: str, iters: int, sync, out):
    _use(impl)
    os.environ.setdefault("MF_DEVICE_BACKEND", "none")   # this repository's module: no GPU involved in this configuration
    import numpy as np
    import memfabric_hybrid as mf
    from memfabric_hybrid import bm
    mf.set_log_level(3)
    assert mf.initialize() == 0
    cfg = bm.BmConfig()
    cfg.auto_ranking = False
    cfg.rank_id = rank
    cfg.start_store = rank == 0
    assert bm.initialize(url, 2, 0, cfg) == 0, mf.get_last_err_msg()
    h = bm.create2(id=0, local_dram_size=64 * MIB, max_dram_size=64 * MIB, data_op_type=bm.BmDataOpType.HOST_SHM)
    assert h.join() == 0, mf.get_last_err_msg()
    sync.wait()
    peer = 1 - rank
    theirs = h.peer_rank_ptr(peer, bm.BmMemType.HOST)
    assert theirs != 0
    rows = []
    rng = np.random.default_rng(100 + rank)
    for size in SIZES:
        src = rng.integers(0, 256, size, dtype=np.uint8)
        back = np.zeros(size, dtype=np.uint8)
        slots = (64 * MIB) // size
        n = max(8, min(iters, 4096))
        # correctness first: put into the peer's slice, get it back, compare CRC32
        assert h.copy_data(src.ctypes.data, theirs, size, bm.BmCopyType.H2G, 0) == 0, mf.get_last_err_msg()
        assert h.copy_data(theirs, back.ctypes.data, size, bm.BmCopyType.G2H, 0) == 0, mf.get_last_err_msg()
        ok = zlib.crc32(src.tobytes()) == zlib.crc32(back.tobytes())
        sync.wait()
        t0 = time.perf_counter()
        for i in range(n):
            h.copy_data(src.ctypes.data, theirs + (i % slots) * size, size, bm.BmCopyType.H2G, 0)
        put = time.perf_counter() - t0
        sync.wait()
        t0 = time.perf_counter()
        for i in range(n):
            h.copy_data(theirs + (i % slots) * size, back.ctypes.data, size, bm.BmCopyType.G2H, 0)
        get = time.perf_counter() - t0
        sync.wait()
        rows.append({"bytes": size, "crc_ok": bool(ok), "calls": n, "lh2gh_us": round(put / n * 1e6, 2), "lh2gh_GBps": round(size * n / put / 1e9, 2),
                     "gh2lh_us": round(get / n * 1e6, 2), "gh2lh_GBps": round(size * n / get / 1e9, 2)})
    assert h.leave() == 0
    sync.wait()
    h.destroy()
    bm.uninitialize(0)
    mf.uninitialize()
    out.put((rank, rows))


def run(impl: str, iters: int = 512, timeout: float = 300.0) -> dict:
    """Runs both ranks as child processes and returns {"impl", "rows": [per size, the slower rank's numbers]}."""
    if impl == "reference" and not os.path.isdir(os.path.join(HERE, "_ref", "memfabric_hybrid")):
        return {"impl": impl, "unavailable": "baseline/_ref/memfabric_hybrid is missing (build the reference with -DXPU_TYPE=NONE first)"}
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    url = f"tcp://127.0.0.1:{s.getsockname()[1]}"
    s.close()
    ctx = mp.get_context("spawn")
    sync, out = ctx.Barrier(2), ctx.Queue()
    procs = [ctx.Process(target=_rank, args=(r, impl, url, iters, sync, out)) for r in range(2)]
    for p in procs:
        p.start()
    res = {}
    deadline = time.time() + timeout
    try:
        while len(res) < 2 and time.time() < deadline:
            try:
                r, rows = out.get(timeout=1.0)
                res[r] = rows
            except Exception:  # noqa: BLE001  (queue.Empty)
                if any(p.exitcode not in (None, 0) for p in procs):
                    break
    finally:
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
    if len(res) < 2:
        return {"impl": impl, "unavailable": f"a rank failed (exit codes {[p.exitcode for p in procs]})"}
    rows = []
    for a, b in zip(res[0], res[1]):
        rows.append({"bytes": a["bytes"], "crc_ok": a["crc_ok"] and b["crc_ok"], "calls": a["calls"],
                     "lh2gh_us": max(a["lh2gh_us"], b["lh2gh_us"]), "lh2gh_GBps": min(a["lh2gh_GBps"], b["lh2gh_GBps"]),
                     "gh2lh_us": max(a["gh2lh_us"], b["gh2lh_us"]), "gh2lh_GBps": min(a["gh2lh_GBps"], b["gh2lh_GBps"])})
    return {"impl": impl, "config": "2 processes, 64 MiB pooled DRAM each, HOST_SHM, copy_data H2G / G2H to and from the peer's slice, CRC32 checked",
            "rows": rows}


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--iters", type=int, default=512)
    a = ap.parse_args()
    print(json.dumps(run(a.impl, a.iters)))
