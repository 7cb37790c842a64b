"""Two ranks share a pooled-DRAM BigMemory object and copy between their slices while each serves its metrics in the
Prometheus text format (GET /metrics): the trace-point table (calls, failures, time, latency histogram per operation),
the pool's copy counters and its capacity. Every rank then scrapes its own endpoint, as Prometheus would with
``prometheus.yaml`` of this folder, and prints the figures the panels of ``grafana_dashboard.json`` are built on.
Works without a GPU.

    python examples/memory_pool/05_observability/metrics_endpoint.py [--port 9464] [--hold SECONDS]

``--hold`` keeps the endpoints up (ports 9464 and 9465 by default) for a real Prometheus to scrape.
"""
import argparse
import os
import sys
import tempfile
import time
import urllib.request

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))
import _launch  # noqa: E402

MiB = 1 << 20


def main(rank: int, world: int, url: str, base_port: int, hold: float) -> dict:
    import memfabric_hybrid as mf
    from memfabric_hybrid import bm
    from memfabric_hybrid_b200.utils import metrics
    os.environ["MF_PTRACER_ENABLE"] = "1"                   # the trace-point table; its file goes to MF_PTRACER_DIR every 10 s
    os.environ.setdefault("MF_PTRACER_DIR", tempfile.gettempdir())
    assert mf.initialize() == 0
    cfg = bm.BmConfig()
    cfg.rank_id = rank
    cfg.start_store = rank == 0
    cfg.set_nic("tcp://127.0.0.1:1234")
    assert bm.initialize(store_url=url, world_size=world, device_id=0, config=cfg) == 0, mf.get_last_err_msg()
    h = bm.create2(id=0, local_dram_size=32 * MiB, max_dram_size=32 * MiB, data_op_type=bm.BmDataOpType.HOST_SHM)
    assert h.join() == 0
    metrics.register_pool("kv", h)
    port = metrics.serve(base_port + rank if base_port else 0)
    peer = (rank + 1) % world
    mine, theirs = h.peer_rank_ptr(rank, bm.BmMemType.HOST), h.peer_rank_ptr(peer, bm.BmMemType.HOST)
    src = np.full(1 * MiB, rank + 1, dtype=np.uint8)
    deadline = time.time() + 30
    while h.copy_data(src.ctypes.data, theirs, src.nbytes, bm.BmCopyType.H2G, 0) != 0:      # until the peer has joined
        assert time.time() < deadline, mf.get_last_err_msg()
        time.sleep(0.05)
    mf.get_and_clear_last_err_msg()
    for i in range(32):                                                                         # some traffic to look at
        assert h.copy_data(mine, mine + 8 * MiB, 256 * 1024, bm.BmCopyType.G2G, 0) == 0
        srcs = [mine + j * 4096 for j in range(16)]
        dsts = [mine + 16 * MiB + j * 4096 for j in range(16)]
        assert h.copy_data_batch(srcs, dsts, [4096] * 16, 16, bm.BmCopyType.G2G, 0) == 0, mf.get_last_err_msg()
    body = urllib.request.urlopen(f"http://127.0.0.1:{port}/metrics", timeout=10).read().decode()
    figures = {}
    for line in body.splitlines():
        if line.startswith("#"):
            continue
        name, value = line.rsplit(" ", 1)
        figures[name] = float(value)
    batch = 'point="TP_BM_COPY_BATCH"'
    out = {"port": port, "families": sorted({n.split("{")[0] for n in figures}),
           "batch_calls": figures.get(f"mf_trace_calls_total{{{batch}}}", 0.0),
           "batch_mean_us": 1e6 * figures.get(f"mf_trace_seconds_total{{{batch}}}", 0.0) / max(1.0, figures.get(f"mf_trace_calls_total{{{batch}}}", 0.0)),
           "capacity": figures.get('mf_pool_local_bytes{mem="host",pool="kv"}', 0.0)}
    if hold > 0:
        print(f"rank {rank}: serving http://127.0.0.1:{port}/metrics for {hold:.0f} s", flush=True)
        time.sleep(hold)
    metrics.unregister_pool("kv")
    metrics.stop()
    h.leave()
    if rank == 0:
        time.sleep(1.0)
    h.destroy()
    bm.uninitialize()
    mf.uninitialize()
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--port", type=int, default=0, help="first metrics port (rank r serves on port + r); 0: any free port")
    ap.add_argument("--hold", type=float, default=0.0, help="seconds to keep the endpoints up after the self-scrape")
    a = ap.parse_args()
    res = _launch.run(main, 2, f"tcp://127.0.0.1:{_launch.free_port()}", a.port, a.hold, timeout=180 + a.hold)
    for r, o in enumerate(res):
        print(f"rank {r}: port {o['port']}, {int(o['batch_calls'])} batched copies, mean {o['batch_mean_us']:.1f} us, "
              f"pool capacity {int(o['capacity']) >> 20} MiB, {len(o['families'])} metric families")
    ok = all(o["batch_calls"] >= 32 and o["capacity"] == 32 * MiB and "mf_trace_duration_seconds_bucket" in o["families"] for o in res)
    print("ok" if ok else "mismatch")
    sys.exit(0 if ok else 1)
