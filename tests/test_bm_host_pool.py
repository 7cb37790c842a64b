"""Host-DRAM pool over the local TCP config store, no GPU: the plumbing configuration.

Two processes each contribute 64 MiB to one GVA range; seeded uint8 buffers of 4 KiB-8 MiB are copied
local-host -> pooled-host (own and peer slot) and pooled-host -> local-host across ranks and verified
by CRC32. Oracle style of the reference's benchmark (benchmark/bm/band_width_calculator.cpp:330-362)."""
import ctypes as C
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


def _rank_56(rank, world, url, sync):
    """Two of 1 024 ranks of a pool whose ranks may grow to 1 TiB each: a 1 PiB window that no process could map."""
    import memfabric_hybrid as mf
    from memfabric_hybrid import bm
    WORLD, TiB = 1024, 1 << 40
    assert mf.initialize() == 0
    cfg = bm.BmConfig()
    cfg.rank_id = rank
    cfg.start_store = rank == 0
    cfg.operation_timeout = 30
    assert bm.initialize(url, WORLD, 0, cfg) == 0, mf.get_last_err_msg()
    # without the switch the window is refused with a reason
    try:
        bm.create2(id=1, local_dram_size=16 * MiB, max_dram_size=TiB, data_op_type=bm.BmDataOpType.HOST_SHM)
        raise AssertionError("a 1 PiB window was accepted without 56-bit addresses")
    except RuntimeError:
        mf.get_and_clear_last_err_msg()
    h = bm.create2(id=0, local_dram_size=16 * MiB, max_dram_size=TiB, data_op_type=bm.BmDataOpType.HOST_SHM, enable_56bits_gva=True)
    assert h.join() == 0, mf.get_last_err_msg()
    sync.wait(60)
    me, peer = h.peer_rank_ptr(rank, bm.BmMemType.HOST), h.peer_rank_ptr(1 - rank, bm.BmMemType.HOST)
    last = h.peer_rank_ptr(WORLD - 1, bm.BmMemType.HOST)
    assert me >= 1 << 55 and last < 1 << 56 and abs(peer - me) == TiB and last - h.peer_rank_ptr(0, bm.BmMemType.HOST) == (WORLD - 1) * TiB
    assert h.get_rank_id_by_gva(peer + 12345) == 1 - rank and h.get_rank_id_by_gva(last + 5) == WORLD - 1
    assert h.local_mem_size(bm.BmMemType.HOST) == 16 * MiB
    rng = np.random.default_rng(100 + rank)
    src = rng.integers(0, 256, 3 * MiB, dtype=np.uint8)
    # the deadline covers the time the peer needs to appear (joining is dynamic)
    import time
    end = time.time() + 30
    while h.copy_data(src.ctypes.data, peer + 4 * MiB, src.nbytes, bm.BmCopyType.H2G, 0) != 0:     # host -> peer's slice
        assert time.time() < end, mf.get_last_err_msg()
        time.sleep(0.05)
    mf.get_and_clear_last_err_msg()
    sync.wait(60)
    want = np.random.default_rng(100 + (1 - rank)).integers(0, 256, 3 * MiB, dtype=np.uint8)
    # pooled -> pooled inside this rank's slice (batched), then out to host memory
    n = 6
    rc = h.copy_data_batch([me + 4 * MiB + i * (MiB // 2) for i in range(n)], [me + 8 * MiB + i * (MiB // 2) for i in range(n)],
                           [MiB // 2] * n, n, bm.BmCopyType.G2G, 0)
    assert rc == 0, mf.get_last_err_msg()
    dst = np.empty(3 * MiB, dtype=np.uint8)
    assert h.copy_data(me + 8 * MiB, dst.ctypes.data, dst.nbytes, bm.BmCopyType.G2H, 0) == 0, mf.get_last_err_msg()
    assert np.array_equal(dst, want)
    # pull from the peer's slice what this rank wrote there
    back = np.empty(3 * MiB, dtype=np.uint8)
    assert h.copy_data(peer + 4 * MiB, back.ctypes.data, back.nbytes, bm.BmCopyType.G2H, 0) == 0 and np.array_equal(back, src)
    # the 56-bit address is a number; gva_to_va gives where the byte lives in this process
    va = h.gva_to_va(me + 8 * MiB + 17)
    assert 0 < va < 1 << 47 and np.ctypeslib.as_array((C.c_uint8 * 4).from_address(va)).tolist() == want[17:21].tolist()
    # out of the mapped part of a slot, a rank that is not there, past the window: refused
    assert h.copy_data(me + 16 * MiB, dst.ctypes.data, 16, bm.BmCopyType.G2H, 0) != 0
    assert h.copy_data(h.peer_rank_ptr(7, bm.BmMemType.HOST), dst.ctypes.data, 16, bm.BmCopyType.G2H, 0) != 0
    assert h.copy_data(last + TiB + 4096, dst.ctypes.data, 16, bm.BmCopyType.G2H, 0) != 0
    mf.get_and_clear_last_err_msg()
    sync.wait(60)
    assert h.leave() == 0
    sync.wait(60)
    h.destroy()
    bm.uninitialize(0)
    mf.uninitialize()
    return True


def test_56_bit_addresses_for_a_window_larger_than_the_address_space(store_url):
    assert run_ranks(_rank_56, 2, (store_url,), timeout=120, with_barrier=True) == [True, True]
