"""A rank grows its slice of a pooled-DRAM object while the pool is in use: the peers learn of it through the
group's update event (handled inside the library) and the new range becomes addressable at the same global address on every rank. Works without a GPU.
The flow of the reference's examples/memory_pool/04_features/02_extend_local_mem example.

    python examples/memory_pool/04_extend_local_mem.py
"""
import os
import sys
import time

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import _launch  # noqa: E402

MiB = 1 << 20


def _retry(fn, what, seconds=30):
    """Joining and extending are dynamic: a range is usable once the owner's event has reached this rank."""
    import memfabric_hybrid as mf
    deadline = time.time() + seconds
    while fn() != 0:
        assert time.time() < deadline, f"{what}: {mf.get_last_err_msg()}"
        time.sleep(0.05)
    mf.get_and_clear_last_err_msg()


def main(rank: int, world: int, url: str) -> str:
    import memfabric_hybrid as mf
    from memfabric_hybrid import bm
    assert mf.initialize() == 0
    cfg = bm.BmConfig()
    cfg.rank_id = rank
    cfg.start_store = rank == 0
    assert bm.initialize(store_url=url, world_size=world, device_id=0, config=cfg) == 0, mf.get_last_err_msg()
    # every rank may grow to 32 MiB (the slot of the address map) and starts with 8 MiB
    h = bm.create2(id=0, local_dram_size=8 * MiB, max_dram_size=32 * MiB, data_op_type=bm.BmDataOpType.HOST_SHM)
    assert h.join() == 0
    peer = 1 - rank
    theirs = h.peer_rank_ptr(peer, bm.BmMemType.HOST)
    mine = h.peer_rank_ptr(rank, bm.BmMemType.HOST)
    src = np.full(4096, 10 + rank, dtype=np.uint8)
    _retry(lambda: h.copy_data(src.ctypes.data, theirs + 1 * MiB, 4096, bm.BmCopyType.H2G, 0), "first copy to the peer")
    # beyond the 8 MiB the peer contributed so far: refused
    assert h.copy_data(src.ctypes.data, theirs + 12 * MiB, 4096, bm.BmCopyType.H2G, 0) != 0
    mf.get_and_clear_last_err_msg()
    assert h.local_mem_size(bm.BmMemType.HOST) == 8 * MiB
    if rank == 0:
        assert h.extend_local_mem(bm.BmMemType.HOST, 8 * MiB) == 0, mf.get_last_err_msg()
        assert h.local_mem_size(bm.BmMemType.HOST) == 16 * MiB
        # wait for the peer's mark inside the new range
        got = np.zeros(4096, dtype=np.uint8)
        deadline = time.time() + 30
        while True:
            assert h.copy_data(mine + 12 * MiB, got.ctypes.data, 4096, bm.BmCopyType.G2H, 0) == 0, mf.get_last_err_msg()
            if (got == 11).all():
                break
            assert time.time() < deadline, "the peer never wrote into the extended range"
            time.sleep(0.05)
    else:
        _retry(lambda: h.copy_data(src.ctypes.data, theirs + 12 * MiB, 4096, bm.BmCopyType.H2G, 0), "copy into the extended range")
    time.sleep(0.5)
    h.leave()
    if rank == 0:
        time.sleep(1.0)                          # this rank hosts the config store: it leaves the stage last
    h.destroy()
    bm.uninitialize()
    mf.uninitialize()
    return "ok"


if __name__ == "__main__":
    res = _launch.run(main, 2, f"tcp://127.0.0.1:{_launch.free_port()}")
    print(res)
    sys.exit(0 if all(r == "ok" for r in res) else 1)
