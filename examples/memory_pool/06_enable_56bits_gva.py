"""A pool whose address window is larger than a process can map: 1 024 ranks that may each grow to 1 TiB of pooled DRAM
(1 PiB in total), of which two ranks run here with 16 MiB each. With ``enable_56bits_gva`` the addresses handed out by
``peer_rank_ptr`` are 56-bit numbers that name (rank, offset); they are passed to the copy calls and never dereferenced.
``gva_to_va`` tells where a byte of the pool is mapped in this process. Works without a GPU. The flow of the reference's
examples/memory_pool/04_features/03_enable_56bits_gva example.

    python examples/memory_pool/06_enable_56bits_gva.py
"""
import ctypes
import os
import sys
import time

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import _launch  # noqa: E402

MiB, TiB, WORLD = 1 << 20, 1 << 40, 1024


def main(rank: int, world: int, url: str) -> str:
    import memfabric_hybrid as mf
    from memfabric_hybrid import bm
    assert mf.initialize() == 0
    cfg = bm.BmConfig()
    cfg.rank_id = rank
    cfg.start_store = rank == 0
    cfg.set_nic("tcp://127.0.0.1:1234")
    assert bm.initialize(store_url=url, world_size=WORLD, device_id=0, config=cfg) == 0, mf.get_last_err_msg()
    h = bm.create2(id=0, local_dram_size=16 * MiB, max_dram_size=TiB, data_op_type=bm.BmDataOpType.HOST_SHM, enable_56bits_gva=True)
    assert h.join() == 0
    peer = 1 - rank
    mine, theirs = h.peer_rank_ptr(rank, bm.BmMemType.HOST), h.peer_rank_ptr(peer, bm.BmMemType.HOST)
    last = h.peer_rank_ptr(WORLD - 1, bm.BmMemType.HOST)
    src = np.full(2 * MiB, rank + 1, dtype=np.uint8)
    deadline = time.time() + 30
    while h.copy_data(src.ctypes.data, theirs, src.nbytes, bm.BmCopyType.H2G, 0) != 0:          # until the peer has joined
        assert time.time() < deadline, mf.get_last_err_msg()
        time.sleep(0.05)
    mf.get_and_clear_last_err_msg()
    time.sleep(0.5)
    dst = np.zeros(2 * MiB, dtype=np.uint8)
    assert h.copy_data(mine, dst.ctypes.data, dst.nbytes, bm.BmCopyType.G2H, 0) == 0              # what the peer wrote here
    va = h.gva_to_va(mine + 100)
    seen = ctypes.c_uint8.from_address(va).value
    ok = bool((dst == peer + 1).all()) and seen == peer + 1 and mine >= 1 << 55 and last - mine == (WORLD - 1 - rank) * TiB
    if rank == 0:
        print(f"rank 0's slice: global {mine:#x}, mapped at {va - 100:#x}; last rank's slice starts at {last:#x}")
    h.leave()
    if rank == 0:
        time.sleep(1.0)
    h.destroy()
    bm.uninitialize()
    mf.uninitialize()
    return "ok" if ok else "mismatch"


if __name__ == "__main__":
    res = _launch.run(main, 2, f"tcp://127.0.0.1:{_launch.free_port()}")
    print(res)
    sys.exit(0 if all(r == "ok" for r in res) else 1)
