"""Two ranks, one pooled-DRAM BigMemory object: host -> pool (own and peer slice) -> pool -> host, then leave.
Works without a GPU. The flow of the reference's
examples/memory_pool/02_scale_out/01_single_node_multi_device_dram example, with the same calls.

    python examples/memory_pool/01_two_rank_dram_pool.py
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
    cfg.rank_id = rank
    cfg.start_store = rank == 0                      # rank 0 hosts the config store
    cfg.set_nic("tcp://127.0.0.1:1234")
    assert bm.initialize(store_url=url, world_size=world, device_id=0, config=cfg) == 0, mf.get_last_err_msg()
    h = bm.create2(id=0, local_dram_size=32 * MiB, max_dram_size=32 * MiB, data_op_type=bm.BmDataOpType.HOST_SHM)
    assert h.join() == 0
    import time
    peer = (rank + 1) % world
    mine, theirs = h.peer_rank_ptr(rank, bm.BmMemType.HOST), h.peer_rank_ptr(peer, bm.BmMemType.HOST)
    src = np.full(1 * MiB, rank + 1, dtype=np.uint8)
    # joining is dynamic: the peer's slice becomes reachable once the peer has joined, so the first copy is retried
    deadline = time.time() + 30
    while h.copy_data(src.ctypes.data, theirs, src.nbytes, bm.BmCopyType.H2G, 0) != 0:          # host -> peer's slice
        assert time.time() < deadline, mf.get_last_err_msg()
        time.sleep(0.05)
    mf.get_and_clear_last_err_msg()
    time.sleep(0.5)                                                                                 # both sides done writing
    assert h.copy_data(mine, mine + 8 * MiB, src.nbytes, bm.BmCopyType.G2G, 0) == 0              # pool -> pool
    dst = np.zeros(1 * MiB, dtype=np.uint8)
    assert h.copy_data(mine + 8 * MiB, dst.ctypes.data, dst.nbytes, bm.BmCopyType.G2H, 0) == 0    # pool -> host
    ok = bool((dst == peer_value(rank, world)).all())
    h.leave()
    if rank == 0:
        time.sleep(1.0)                              # this rank hosts the config store: it leaves the stage last
    h.destroy()
    bm.uninitialize()
    mf.uninitialize()
    assert mf.get_last_err_msg() == ""
    return "ok" if ok else "mismatch"


def peer_value(rank, world):
    return (rank - 1) % world + 1                    # the rank that wrote into my slice


if __name__ == "__main__":
    res = _launch.run(main, 2, f"tcp://127.0.0.1:{_launch.free_port()}")
    print(res)
    sys.exit(0 if all(r == "ok" for r in res) else 1)
