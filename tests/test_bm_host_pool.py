"""Host-DRAM pool over the local TCP config store, no GPU: the plumbing configuration.

Two processes each contribute 64 MiB to one GVA range; seeded uint8 buffers of 4 KiB-8 MiB are copied
local-host -> pooled-host (own and peer slot) and pooled-host -> local-host across ranks and verified
by CRC32. Oracle style of the reference's benchmark (benchmark/bm/band_width_calculator.cpp:330-362)."""
import zlib

import numpy as np

from mp_util import run_ranks

MiB = 1 << 20
SIZES = [4 << 10, 64 << 10, 1 * MiB, 8 * MiB]


def _rank(rank, world, url, sync):
    import memfabric_hybrid as mf
    from memfabric_hybrid import bm
    assert mf.initialize() == 0
    cfg = bm.BmConfig()
    cfg.rank_id = rank
    cfg.start_store = rank == 0
    cfg.operation_timeout = 30
    assert bm.initialize(url, world, 0, cfg) == 0, mf.get_last_err_msg()
    assert bm.bm_rank_id() == rank
    h = bm.create2(id=0, local_dram_size=64 * MiB, max_dram_size=64 * MiB, data_op_type=bm.BmDataOpType.HOST_SHM)
    assert h.join() == 0, mf.get_last_err_msg()
    sync.wait(60)  # join is dynamic: wait until both ranks are members
    me = h.peer_rank_ptr(rank, bm.BmMemType.HOST)
    peer = h.peer_rank_ptr(1 - rank, bm.BmMemType.HOST)
    assert me and peer and abs(peer - me) == 64 * MiB
    assert h.get_rank_id_by_gva(peer + 5) == 1 - rank
    assert h.local_mem_size(bm.BmMemType.HOST) == 64 * MiB
    crcs = {}
    off = 0
    rng = np.random.default_rng(rank)  # seed = rank so that the two directions carry different data
    for sz in SIZES:
        src = rng.integers(0, 256, sz, dtype=np.uint8)
        crcs[sz] = zlib.crc32(src.tobytes())
        # LH -> GH into the PEER's slot (remote write through the mapping)
        assert h.copy_data(src.ctypes.data, peer + off, sz, bm.BmCopyType.H2GH, 0) == 0, mf.get_last_err_msg()
        off += sz
    sync.wait(60)  # both ranks done writing before anybody reads
    # GH -> LH from OUR slot: what the peer wrote (seeded with the peer's rank)
    peer_rng = np.random.default_rng(1 - rank)
    off = 0
    for sz in SIZES:
        want = zlib.crc32(peer_rng.integers(0, 256, sz, dtype=np.uint8).tobytes())
        dst = np.empty(sz, dtype=np.uint8)
        assert h.copy_data(me + off, dst.ctypes.data, sz, bm.BmCopyType.GH2H, 0) == 0, mf.get_last_err_msg()
        assert zlib.crc32(dst.tobytes()) == want, f"size {sz}"
        off += sz
    # batched G2G pull of everything from the peer's slot... which holds what WE wrote
    n = len(SIZES)
    offs = np.cumsum([0] + SIZES[:-1]).tolist()
    stage = 32 * MiB
    rc = h.copy_data_batch([peer + o for o in offs], [me + stage + o for o in offs], SIZES, n, bm.BmCopyType.G2G, 0)
    assert rc == 0, mf.get_last_err_msg()
    for o, sz in zip(offs, SIZES):
        dst = np.empty(sz, dtype=np.uint8)
        assert h.copy_data(me + stage + o, dst.ctypes.data, sz, bm.BmCopyType.G2H, 0) == 0
        assert zlib.crc32(dst.tobytes()) == crcs[sz]
    # an address outside the pool is refused, not followed
    bad = h.copy_data(me + 64 * MiB * 2 + 4096, dst.ctypes.data, 16, bm.BmCopyType.GH2H, 0)
    assert bad != 0
    mf.get_and_clear_last_err_msg()
    sync.wait(60)
    rc = h.leave()
    assert rc == 0, f"leave returned {rc}: {mf.get_last_err_msg()}"
    sync.wait(60)  # rank 0 hosts the config store: it must not tear it down while the peer is still leaving
    h.destroy()
    bm.uninitialize(0)
    mf.uninitialize()
    return True


def test_two_rank_dram_pool(store_url):
    assert run_ranks(_rank, 2, (store_url,), timeout=120, with_barrier=True) == [True, True]
