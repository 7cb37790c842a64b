"""Batched copies between host buffers and the pool, with the host buffers registered up front so that the
per-copy address bookkeeping is skipped (examples/memory_pool/03_optimization/01_copy_data_batch and
02_register of the reference). One rank; works without a GPU.

    python examples/memory_pool/02_copy_data_batch_and_register.py
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import _launch  # noqa: E402

MiB = 1 << 20


def main(rank: int, world: int, url: str) -> str:
    import memfabric_hybrid as mf
    from memfabric_hybrid import bm
    assert mf.initialize() == 0
    cfg = bm.BmConfig()
    cfg.rank_id, cfg.start_store = rank, True
    assert bm.initialize(url, world, 0, cfg) == 0
    h = bm.create(id=0, local_dram_size=64 * MiB, local_hbm_size=0, data_op_type=bm.BmDataOpType.HOST_SHM)
    assert h.join() == 0
    base = h.peer_rank_ptr(rank, bm.BmMemType.HOST)
    n, blk = 64, 128 << 10
    src = np.random.default_rng(0).integers(0, 256, n * blk, dtype=np.uint8)
    dst = np.zeros_like(src)
    assert h.register(src.ctypes.data, src.nbytes) == 0 and h.register(dst.ctypes.data, dst.nbytes) == 0
    srcs = [src.ctypes.data + i * blk for i in range(n)]
    pool = [base + i * blk for i in range(n)]
    back = [dst.ctypes.data + i * blk for i in range(n)]
    assert h.copy_data_batch(srcs, pool, [blk] * n, n, bm.BmCopyType.H2G, 0) == 0
    assert h.copy_data_batch(pool, back, [blk] * n, n, bm.BmCopyType.G2H, 0) == 0
    ok = bool((src == dst).all())
    h.unregister(src.ctypes.data)
    h.unregister(dst.ctypes.data)
    h.leave()
    h.destroy()
    bm.uninitialize()
    mf.uninitialize()
    return "ok" if ok else "mismatch"


if __name__ == "__main__":
    res = _launch.run(main, 1, f"tcp://127.0.0.1:{_launch.free_port()}")
    print(res)
    sys.exit(0 if res == ["ok"] else 1)
