"""The HBM-pool code path (VMM segment, fd channel, batch descriptors, partial results) on a machine
without a GPU, against the fake device backend whose "device memory" is memfd-backed host memory."""
import numpy as np

from conftest import free_port
from mp_util import run_ranks

MiB = 1 << 20


def _rank(rank, world, url, sync):
    import memfabric_hybrid as mf
    from memfabric_hybrid import bm
    assert mf.initialize() == 0
    cfg = bm.BmConfig()
    cfg.auto_ranking = True        # ranks come from the store, every process races to host it
    cfg.start_store = True
    cfg.operation_timeout = 30
    assert bm.initialize(url, world, 0, cfg) == 0, mf.get_last_err_msg()
    me = bm.bm_rank_id()
    assert me in (0, 1)
    h = bm.create2(id=3, local_dram_size=4 * MiB, max_dram_size=8 * MiB, local_hbm_size=8 * MiB, max_hbm_size=16 * MiB)
    events = []
    h.set_group_event_handler(lambda r, ev: events.append((r, int(ev))))
    assert h.join() == 0, mf.get_last_err_msg()
    sync.wait(60)
    peer = 1 - me
    pdev = h.peer_rank_ptr(peer, bm.BmMemType.DEVICE)
    mdev = h.peer_rank_ptr(me, bm.BmMemType.DEVICE)
    assert abs(pdev - mdev) == 16 * MiB
    src = np.random.default_rng(me).integers(0, 256, 2 * MiB, dtype=np.uint8)
    n, seg = 16, 128 * 1024
    rc = h.copy_data_batch([src.ctypes.data + i * seg for i in range(n)], [pdev + i * seg for i in range(n)], [seg] * n, n,
                           bm.BmCopyType.H2G, 0)
    assert rc == 0, mf.get_last_err_msg()
    sync.wait(60)
    got = np.zeros(2 * MiB, dtype=np.uint8)
    assert h.copy_data(mdev, got.ctypes.data, 2 * MiB, bm.BmCopyType.G2H, 0) == 0, mf.get_last_err_msg()
    want = np.random.default_rng(peer).integers(0, 256, 2 * MiB, dtype=np.uint8)
    assert np.array_equal(got, want)
    # beyond the 8 MiB that the peer contributed (its slot is 16 MiB): refused
    assert h.copy_data(src.ctypes.data, pdev + 9 * MiB, 4096, bm.BmCopyType.H2G, 0) != 0
    mf.get_and_clear_last_err_msg()
    # a batch with one bad destination: the good items are copied and every item reports its own result
    rc, res = h.copy_data_batch_partial_succeed([src.ctypes.data, src.ctypes.data + 4096, src.ctypes.data + 8192],
                                                [pdev + 4 * MiB, pdev + 9 * MiB, pdev + 4 * MiB + 8192], [4096] * 3, 3,
                                                bm.BmCopyType.H2G, 0)
    assert rc != 0 and res[0] == 0 and res[1] != 0 and res[2] == 0, (rc, res)
    mf.get_and_clear_last_err_msg()
    back = np.zeros(4096, dtype=np.uint8)
    assert h.copy_data(pdev + 4 * MiB + 8192, back.ctypes.data, 4096, bm.BmCopyType.G2H, 0) == 0
    assert np.array_equal(back, src[8192:12288])
    # the peer extends its slice; after the update the same address is valid
    sync.wait(60)
    if me == 0:
        assert h.extend_local_mem(bm.BmMemType.DEVICE, 4 * MiB) == 0, mf.get_last_err_msg()
    sync.wait(60)
    if me == 1:
        assert h.copy_data(src.ctypes.data, pdev + 9 * MiB, 4096, bm.BmCopyType.H2G, 0) == 0, mf.get_last_err_msg()
    sync.wait(60)
    # rank 1 leaves: rank 0 gets a LEAVE event and copies to rank 1 are refused afterwards
    if me == 1:
        assert h.leave() == 0
    sync.wait(60)
    if me == 0:
        import time
        t0 = time.time()
        while (1, 1) not in events and time.time() - t0 < 20:
            time.sleep(0.01)
        assert (1, 1) in events, events
        assert h.copy_data(src.ctypes.data, pdev, 4096, bm.BmCopyType.H2G, 0) != 0
        mf.get_and_clear_last_err_msg()
        # the quantising copy checks its pooled addresses like every other copy: the slice of the rank that left is
        # refused as "not connected" instead of being handed to the kernel
        import torch
        row = torch.randn(128).to(torch.bfloat16)
        rc = h.quant_copy_batch([row.data_ptr()], [pdev], [256], [pdev + MiB], 64)
        assert rc == -2014, rc
        assert "not mapped" in mf.get_and_clear_last_err_msg()
        assert h.leave() == 0
    sync.wait(60)  # whichever process hosts the config store must not tear it down while the other still leaves
    h.destroy()
    bm.uninitialize(0)
    mf.uninitialize()
    return me


def test_fake_device_two_ranks():
    url = f"tcp://127.0.0.1:{free_port()}"
    ranks = run_ranks(_rank, 2, (url,), timeout=180, env={"MF_DEVICE_BACKEND": "fake"}, with_barrier=True)
    assert sorted(ranks) == [0, 1]


def _quant_rank(rank, world, url):
    import torch
    import memfabric_hybrid as mf
    from memfabric_hybrid import bm
    assert mf.initialize() == 0
    cfg = bm.BmConfig()
    cfg.rank_id, cfg.start_store, cfg.auto_ranking = 0, True, False
    assert bm.initialize(url, 1, 0, cfg) == 0, mf.get_last_err_msg()
    h = bm.create2(id=4, local_dram_size=0, max_dram_size=0, local_hbm_size=8 * MiB, max_hbm_size=8 * MiB)
    assert h.join() == 0, mf.get_last_err_msg()
    base = h.peer_rank_ptr(0, bm.BmMemType.DEVICE)
    rows, unit, cols = 3, 64, 200                                     # 200 = 3 units of 64 + a tail of 8
    x = (torch.randn(rows, cols) * 4).to(torch.bfloat16)
    x[1, :64] = 0
    units = (cols + unit - 1) // unit
    q_at, s_at = base, base + MiB
    rc = h.quant_copy_batch([x[i].data_ptr() for i in range(rows)], [q_at + i * 256 for i in range(rows)], [cols * 2] * rows,
                            [s_at + i * units * 4 for i in range(rows)], unit)
    assert rc == 0, mf.get_last_err_msg()
    q = np.zeros((rows, 256), dtype=np.int8)
    s = np.zeros((rows, units), dtype=np.float32)
    assert h.copy_data(q_at, q.ctypes.data, q.nbytes, bm.BmCopyType.G2H, 0) == 0
    assert h.copy_data(s_at, s.ctypes.data, s.nbytes, bm.BmCopyType.G2H, 0) == 0
    xf = x.float().numpy()
    for i in range(rows):
        for u in range(units):
            seg = xf[i, u * unit:min(cols, (u + 1) * unit)]
            am = np.abs(seg).max()
            if am == 0:
                assert s[i, u] == 1.0 and not q[i, u * unit:u * unit + len(seg)].any()
                continue
            assert abs(s[i, u] - am / 127.0) < 1e-6
            assert np.abs(q[i, u * unit:u * unit + len(seg)] - np.rint(seg * np.float32(127.0 / am))).max() <= 1
    assert not q[:, cols:].any()                                      # nothing written past the row
    # a destination or a factor array that runs past the mapped slice is refused before anything is launched
    assert h.quant_copy_batch([x[0].data_ptr()], [base + 8 * MiB - 64], [cols * 2], [s_at], unit) == -2000
    assert "runs past" in mf.get_and_clear_last_err_msg()
    assert h.quant_copy_batch([x[0].data_ptr()], [q_at], [cols * 2], [base + 8 * MiB - 8], unit) == -2000
    mf.get_and_clear_last_err_msg()
    # a length that would wrap the range check is refused too
    probe = np.zeros(16, dtype=np.uint8)
    assert h.copy_data(base, probe.ctypes.data, (1 << 64) - 8, bm.BmCopyType.G2H, 0) != 0
    mf.get_and_clear_last_err_msg()
    rc, res = h.copy_data_batch_partial_succeed([base], [probe.ctypes.data], [(1 << 64) - 8], 1, bm.BmCopyType.G2H, 0)
    assert rc != 0 and res[0] != 0
    mf.get_and_clear_last_err_msg()
    # the fp8 format needs the device: refused by the host oracle, with a message
    assert h.quant_copy_batch([x[0].data_ptr()], [q_at], [128 * 2], [s_at], 128, fp8=True) != 0
    mf.get_and_clear_last_err_msg()
    h.leave()
    h.destroy()
    bm.uninitialize(0)
    mf.uninitialize()
    return 0


def test_quantising_copy_against_the_host_oracle():
    url = f"tcp://127.0.0.1:{free_port()}"
    assert run_ranks(_quant_rank, 1, (url,), timeout=120, env={"MF_DEVICE_BACKEND": "fake"}) == [0]


def _rank_56(rank, world, url, sync):
    """Windows of 1 024 ranks x 256 GiB of HBM and x 1 TiB of DRAM (two ranks present): 56-bit addresses on the device-memory path."""
    import memfabric_hybrid as mf
    from memfabric_hybrid import bm
    WORLD, TiB = 1024, 1 << 40
    assert mf.initialize() == 0
    cfg = bm.BmConfig()
    cfg.rank_id, cfg.start_store, cfg.auto_ranking = rank, rank == 0, False
    cfg.operation_timeout = 30
    assert bm.initialize(url, WORLD, 0, cfg) == 0, mf.get_last_err_msg()
    h = bm.create2(id=5, local_dram_size=4 * MiB, max_dram_size=TiB, local_hbm_size=8 * MiB, max_hbm_size=TiB // 4, enable_56bits_gva=True)
    assert h.join() == 0, mf.get_last_err_msg()
    sync.wait(60)
    peer = 1 - rank
    mdev, pdev = h.peer_rank_ptr(rank, bm.BmMemType.DEVICE), h.peer_rank_ptr(peer, bm.BmMemType.DEVICE)
    mhost = h.peer_rank_ptr(rank, bm.BmMemType.HOST)
    assert mdev >= 1 << 55 and mhost >= 1 << 55 and abs(pdev - mdev) == TiB // 4 and not (mdev <= mhost < mdev + WORLD * TiB // 4)
    assert h.get_rank_id_by_gva(pdev + 99) == peer
    src = np.random.default_rng(50 + rank).integers(0, 256, 2 * MiB, dtype=np.uint8)
    n, seg = 16, 128 * 1024
    import time
    end = time.time() + 30
    while h.copy_data_batch([src.ctypes.data + i * seg for i in range(n)], [pdev + i * seg for i in range(n)], [seg] * n, n,
                            bm.BmCopyType.H2G, 0) != 0:                      # host -> the peer's device slice, batched
        assert time.time() < end, mf.get_last_err_msg()
        time.sleep(0.05)
    mf.get_and_clear_last_err_msg()
    sync.wait(60)
    want = np.random.default_rng(50 + peer).integers(0, 256, 2 * MiB, dtype=np.uint8)
    # device pool -> device pool (own slice), device pool -> DRAM pool, DRAM pool -> host
    assert h.copy_data_batch([mdev + i * seg for i in range(n)], [mdev + 4 * MiB + i * seg for i in range(n)], [seg] * n, n,
                             bm.BmCopyType.G2G, 0) == 0, mf.get_last_err_msg()
    assert h.copy_data(mdev + 4 * MiB, mhost, 2 * MiB, bm.BmCopyType.G2G, 0) == 0, mf.get_last_err_msg()
    got = np.zeros(2 * MiB, dtype=np.uint8)
    assert h.copy_data(mhost, got.ctypes.data, 2 * MiB, bm.BmCopyType.G2H, 0) == 0, mf.get_last_err_msg()
    assert np.array_equal(got, want)
    # a prepared batch (validated once, launched many times) translates too
    pb = h.prepare_batch([pdev + i * seg for i in range(4)], [mdev + 6 * MiB + i * seg for i in range(4)], [seg] * 4, 4)
    assert h.copy_prepared(pb, bm.BmCopyType.G2G, 0) == 0, mf.get_last_err_msg()
    back = np.zeros(4 * seg, dtype=np.uint8)
    assert h.copy_data(mdev + 6 * MiB, back.ctypes.data, back.nbytes, bm.BmCopyType.G2H, 0) == 0 and np.array_equal(back, src[:4 * seg])
    assert h.copy_data(mdev + 8 * MiB, got.ctypes.data, 16, bm.BmCopyType.G2H, 0) != 0        # past what the rank contributed
    assert h.copy_data(h.peer_rank_ptr(9, bm.BmMemType.DEVICE), got.ctypes.data, 16, bm.BmCopyType.G2H, 0) != 0
    mf.get_and_clear_last_err_msg()
    sync.wait(60)
    assert h.leave() == 0
    sync.wait(60)
    h.destroy()
    bm.uninitialize(0)
    mf.uninitialize()
    return True


def test_fake_device_56_bit_addresses():
    url = f"tcp://127.0.0.1:{free_port()}"
    assert run_ranks(_rank_56, 2, (url,), timeout=180, env={"MF_DEVICE_BACKEND": "fake"}, with_barrier=True) == [True, True]
