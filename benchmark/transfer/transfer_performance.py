"""Transfer-engine performance through the Python API: per-block latency, batched bandwidth and concurrent writers.

Two ranks. Rank 1 ("Decode") owns the config store and registers the destination buffer; rank 0 ("Prefill") writes into it:

    python transfer_performance.py --rank-id 1 --store-url tcp://127.0.0.1:12050 --gpu-id 1 &
    python transfer_performance.py --rank-id 0 --store-url tcp://127.0.0.1:12050 --gpu-id 0 --num-threads 2
    python transfer_performance.py --both --store-url tcp://127.0.0.1:12050          # both ranks from one command

Block sizes 32 KiB .. 16 MiB, 32 blocks per batch (the sweep of the reference's benchmark/transfer/perf_python tool, same
arguments; --npu-id is accepted as an alias of --gpu-id, --data-op-type sdma | rdma select the same NVLink / PCIe path here).
Without a GPU the buffers are host memory. The destination address travels through a small file next to the store port."""
from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

BLOCKS = 32
SIZES = [32 << 10 << i for i in range(10)]   # 32 KiB .. 16 MiB


def _buffers(nbytes: int, gpu: int, fill: int):
    """(tensor or array that owns the memory, address)."""
    try:
        import torch
        if torch.cuda.is_available():
            torch.cuda.set_device(gpu % torch.cuda.device_count())
            t = torch.full((nbytes,), fill, dtype=torch.uint8, device="cuda")
            return t, t.data_ptr(), True
    except ImportError:
        pass
    import numpy as np
    a = np.full(nbytes, fill, dtype=np.uint8)
    return a, a.ctypes.data, False


def _meet(store_url: str) -> str:
    port = store_url.rsplit(":", 1)[-1]
    return os.path.join(tempfile.gettempdir(), f"mf_transfer_perf_{port}.json")


def decode_side(args, max_block: int) -> int:
    from memfabric_hybrid import TransferEngine
    eng = TransferEngine()
    session = args.store_url.split("//", 1)[-1]
    assert eng.initialize(args.store_url, session, "Decode", args.gpu_id) == 0, "initialize failed"
    owner, addr, _ = _buffers(max_block * BLOCKS, args.gpu_id, 0)
    assert eng.register_memory(addr, max_block * BLOCKS) == 0
    meet = _meet(args.store_url)
    with open(meet + ".tmp", "w") as f:
        json.dump({"session": session, "addr": addr}, f)
    os.replace(meet + ".tmp", meet)
    done = meet + ".done"
    deadline = time.time() + args.timeout
    while not os.path.exists(done) and time.time() < deadline:
        time.sleep(0.05)
    ok = os.path.exists(done)
    for p in (meet, done):
        if os.path.exists(p):
            os.remove(p)
    eng.destroy()
    eng.unInitialize()
    del owner
    return 0 if ok else 1


def prefill_side(args, max_block: int) -> int:
    from memfabric_hybrid import TransferEngine
    eng = TransferEngine()
    me = f"127.0.0.1:{20000 + os.getpid() % 20000}"
    assert eng.initialize(args.store_url, me, "Prefill", args.gpu_id) == 0, "initialize failed"
    meet = _meet(args.store_url)
    deadline = time.time() + args.timeout
    while not os.path.exists(meet):
        assert time.time() < deadline, "the receiving rank did not publish its buffer"
        time.sleep(0.05)
    info = json.load(open(meet))
    peer, dst = info["session"], int(info["addr"])
    src_owner, src, on_gpu = _buffers(max_block * BLOCKS, args.gpu_id, 0x5A)
    chk_owner, chk, _ = _buffers(max_block * BLOCKS, args.gpu_id, 0)
    assert eng.register_memory(src, max_block * BLOCKS) == 0 and eng.register_memory(chk, max_block * BLOCKS) == 0
    bad = 0
    rows = []
    for bs in [s for s in SIZES if s <= max_block]:
        srcs = [src + i * bs for i in range(BLOCKS)]
        dsts = [dst + i * bs for i in range(BLOCKS)]
        lens = [bs] * BLOCKS
        # the receiver's registration becomes visible shortly after it starts: the first write is retried
        t_end = time.time() + 30
        while eng.transfer_sync_write(peer, src, dst, bs) != 0:
            assert time.time() < t_end, "write failed"
            time.sleep(0.05)
        # latency of one block
        n = 20
        t0 = time.perf_counter()
        for _ in range(n):
            assert eng.transfer_sync_write(peer, src, dst, bs) == 0
        lat_us = (time.perf_counter() - t0) / n * 1e6
        # bandwidth of batches of 32 blocks
        assert eng.batch_transfer_sync_write(peer, srcs, dsts, lens) == 0
        t0 = time.perf_counter()
        for _ in range(n):
            assert eng.batch_transfer_sync_write(peer, srcs, dsts, lens) == 0
        batch_us = (time.perf_counter() - t0) / n * 1e6
        # concurrent writers, each on its own share of the blocks
        per = max(1, BLOCKS // args.num_threads)
        def worker(k):
            lo = k * per
            for _ in range(n):
                eng.batch_transfer_sync_write(peer, srcs[lo:lo + per], dsts[lo:lo + per], lens[lo:lo + per])
        ths = [threading.Thread(target=worker, args=(k,)) for k in range(args.num_threads)]
        t0 = time.perf_counter()
        for t in ths:
            t.start()
        for t in ths:
            t.join()
        conc_us = (time.perf_counter() - t0) / n * 1e6
        # read back and compare
        assert eng.batch_transfer_sync_read(peer, [chk + i * bs for i in range(BLOCKS)], dsts, lens) == 0
        if on_gpu:
            import torch
            same = bool(torch.equal(chk_owner[:bs * BLOCKS], src_owner[:bs * BLOCKS]))
        else:
            same = bool((chk_owner[:bs * BLOCKS] == src_owner[:bs * BLOCKS]).all())
        bad += not same
        row = {"block_KB": bs >> 10, "latency_us": round(lat_us, 1), "batch32_us": round(batch_us, 1),
               "batch32_GBps": round(bs * BLOCKS / batch_us / 1e3, 2), f"threads{args.num_threads}_GBps": round(per * args.num_threads * bs / conc_us / 1e3, 2),
               "verified": same}
        rows.append(row)
        print(f"Test completed: latency {lat_us:.1f}us, block size {bs >> 10}KB, total size {bs * BLOCKS >> 10}KB , "
              f"throughput {row['batch32_GBps']:.2f} GB/s, {args.num_threads} threads {row[f'threads{args.num_threads}_GBps']:.2f} GB/s, "
              f"verified {'yes' if same else 'NO'}", flush=True)
    open(meet + ".done", "w").write("1")
    time.sleep(0.2)
    eng.destroy()
    eng.unInitialize()
    print(json.dumps({"tool": "transfer_performance", "device": "gpu" if on_gpu else "host", "rows": rows}))
    return 1 if bad else 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rank-id", type=int, default=0)
    ap.add_argument("--store-url", default="tcp://127.0.0.1:12050")
    ap.add_argument("--num-threads", type=int, default=2)
    ap.add_argument("--data-op-type", default="sdma", choices=["sdma", "rdma"])
    ap.add_argument("--gpu-id", "--npu-id", dest="gpu_id", type=int, default=0)
    ap.add_argument("--max-block-kb", type=int, default=16384)
    ap.add_argument("--timeout", type=float, default=300.0)
    ap.add_argument("--both", action="store_true", help="start the receiving rank as a child process, then run the sender")
    args = ap.parse_args()
    max_block = min(16 << 20, max(32 << 10, args.max_block_kb << 10))
    if args.both:
        import subprocess
        child = subprocess.Popen([sys.executable, os.path.abspath(__file__), "--rank-id", "1", "--store-url", args.store_url,
                                  "--gpu-id", str(args.gpu_id + 1), "--max-block-kb", str(args.max_block_kb), "--timeout", str(args.timeout)])
        try:
            rc = prefill_side(args, max_block)
        finally:
            try:
                child.wait(timeout=30)
            except subprocess.TimeoutExpired:
                child.kill()
        return rc or child.returncode or 0
    return decode_side(args, max_block) if args.rank_id == 1 else prefill_side(args, max_block)


if __name__ == "__main__":
    sys.exit(main())
