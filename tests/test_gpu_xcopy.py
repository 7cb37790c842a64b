"""GPU tests of the pooled-HBM copy paths (bit-exact against the source data).

Two processes on ONE device are a valid test of the inter-process mapping (VMM export over the fd
channel, peer mapping, batched kernel) because the copy kernels never wait on one another."""
import zlib

import numpy as np
import pytest

from conftest import free_port
from mp_util import run_ranks

pytestmark = pytest.mark.gpu
MiB = 1 << 20


def test_smoke_single_rank():
    from memfabric_hybrid_b200 import smoke
    smoke.run()


def _two_ranks(rank, world, url, sync):
    import torch
    import memfabric_hybrid as mf
    from memfabric_hybrid import bm
    ndev = torch.cuda.device_count()
    dev_id = rank % ndev
    torch.cuda.set_device(dev_id)
    assert mf.initialize() == 0
    cfg = bm.BmConfig()
    cfg.rank_id = rank
    cfg.start_store = rank == 0
    cfg.operation_timeout = 60
    assert bm.initialize(url, world, dev_id, cfg) == 0, mf.get_last_err_msg()
    h = bm.create2(id=1, local_dram_size=32 * MiB, max_dram_size=32 * MiB, local_hbm_size=128 * MiB, max_hbm_size=128 * MiB)
    assert h.join() == 0, mf.get_last_err_msg()
    sync.wait(120)
    peer = 1 - rank
    g = torch.Generator("cuda").manual_seed(100 + rank)
    x = torch.randint(0, 255, (64 * MiB,), dtype=torch.uint8, device="cuda", generator=g)
    pdev = h.peer_rank_ptr(peer, bm.BmMemType.DEVICE)
    mdev = h.peer_rank_ptr(rank, bm.BmMemType.DEVICE)
    # The pool's internal stream is not ordered with PyTorch's: tensors that a PyTorch kernel fills must be
    # complete before a copy that runs there reads or overwrites them.
    torch.cuda.synchronize()
    # D2RD: odd sizes and offsets on purpose (head/tail paths), plus big aligned segments
    segs = [(0, 1 * MiB), (1 * MiB + 3, 4097), (2 * MiB + 16, 16 * 1024), (3 * MiB, 8 * MiB), (12 * MiB + 1, 777), (16 * MiB, 32 * MiB)]
    srcs = [x.data_ptr() + o for o, _ in segs]
    dsts = [pdev + o for o, _ in segs]
    sizes = [s for _, s in segs]
    assert h.copy_data_batch(srcs, dsts, sizes, len(segs), bm.BmCopyType.L2G, 0) == 0, mf.get_last_err_msg()
    sync.wait(120)
    # what the peer pushed into OUR slice
    gp = torch.Generator("cuda").manual_seed(100 + peer)
    want = torch.randint(0, 255, (64 * MiB,), dtype=torch.uint8, device="cuda", generator=gp)
    got = torch.zeros(64 * MiB, dtype=torch.uint8, device="cuda")
    pulled = torch.zeros(8 * MiB, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    assert h.copy_data_batch([mdev + o for o, _ in segs], [got.data_ptr() + o for o, _ in segs], sizes, len(segs),
                             bm.BmCopyType.G2L, 0) == 0, mf.get_last_err_msg()
    for o, s in segs:
        assert torch.equal(got[o:o + s], want[o:o + s]), f"segment at {o} (+{s}) differs"
    # RD2D pull from the peer's slice (it holds OUR data) and a D2H leg into the pooled DRAM, then GH2H
    assert h.copy_data(pdev + 3 * MiB, pulled.data_ptr(), 8 * MiB, bm.BmCopyType.G2L, 0) == 0, mf.get_last_err_msg()
    assert torch.equal(pulled, x[3 * MiB:11 * MiB])
    mhost = h.peer_rank_ptr(rank, bm.BmMemType.HOST)
    assert h.copy_data(x.data_ptr(), mhost, 8 * MiB, bm.BmCopyType.L2GH, 0) == 0, mf.get_last_err_msg()
    back = np.empty(8 * MiB, dtype=np.uint8)
    assert h.copy_data(mhost, back.ctypes.data, 8 * MiB, bm.BmCopyType.GH2H, 0) == 0
    assert zlib.crc32(back.tobytes()) == zlib.crc32(x[:8 * MiB].cpu().numpy().tobytes())
    # async + wait on the internal stream
    assert h.copy_data(x.data_ptr(), pdev + 48 * MiB, 16 * MiB, bm.BmCopyType.L2G, bm.ASYNC_COPY_FLAG) == 0
    assert h.wait() == 0
    # per-item results: one bad item out of three
    rc, res = h.copy_data_batch_partial_succeed([x.data_ptr(), x.data_ptr(), x.data_ptr()],
                                                [pdev, pdev + 1024 * MiB, pdev + MiB], [4096, 4096, 4096], 3, bm.BmCopyType.L2G, 0)
    assert rc == -2012 and res[0] == 0 and res[1] != 0 and res[2] == 0, (rc, res)
    mf.get_and_clear_last_err_msg()
    st = h.copy_stats()
    sync.wait(120)
    assert h.leave() == 0
    sync.wait(120)  # rank 0 hosts the config store: no teardown while the peer is still leaving
    h.destroy()
    bm.uninitialize(0)
    mf.uninitialize()
    return st["kernel_launches"]


def test_two_process_hbm_pool():
    url = f"tcp://127.0.0.1:{free_port()}"
    launches = run_ranks(_two_ranks, 2, (url,), timeout=300, with_barrier=True)
    assert all(l > 0 for l in launches), f"SM copy kernel did not run: {launches}"


@pytest.mark.parametrize("bulk", [0, 1])
def test_copy_kernels_refuse_descriptors_outside_the_mapped_window(bulk):
    """The debug window of the copy kernels (MF_XCOPY_DEBUG=1 publishes the pool's window; here it is handed in directly):
    a descriptor whose pooled side runs past the mapped part of a slot is skipped before its first access and reported;
    its neighbours are copied."""
    import ctypes as C
    import torch
    from memfabric_hybrid_b200 import _native as N
    cu = N.cuda()
    cu.mf_xcopy_debug_probe.restype = C.c_int
    cu.mf_xcopy_debug_probe.argtypes = [C.POINTER(C.c_uint64), C.c_uint32, C.c_uint64, C.c_uint64, C.c_uint32, C.POINTER(C.c_uint64), C.c_int]
    n = 64 << 10
    src = torch.arange(n, device="cuda", dtype=torch.int32)
    pool = torch.zeros(4 * n, device="cuda", dtype=torch.int32)       # stands for a window of 4 slots of n ints, 3/4 of each mapped
    other = torch.zeros(n, device="cuda", dtype=torch.int32)
    torch.cuda.synchronize()
    slot = n * 4
    base = pool.data_ptr()
    mapped = (C.c_uint64 * 4)(*[slot * 3 // 4] * 4)
    half = n * 2                                                      # bytes of half a slot
    trip = [src.data_ptr(), base, half,                               # into the mapped part of slot 0
            src.data_ptr(), base + slot + slot // 2, half,            # slot 1: starts inside, ends past the mapped 3/4: refused
            src.data_ptr(), other.data_ptr(), half,                   # neither side in the window: taken as given
            src.data_ptr(), base + 4 * slot - 4096, 4096 * 2]         # runs out of the window's last slot: refused
    arr = (C.c_uint64 * len(trip))(*trip)
    rc = cu.mf_xcopy_debug_probe(arr, len(trip) // 3, base, slot, 4, mapped, bulk)
    assert rc == 0x7D1, hex(rc & 0xFFFFFFFF)
    torch.cuda.synchronize()
    q = n // 2
    assert torch.equal(pool[:q], src[:q]) and torch.equal(other[:q], src[:q])
    assert int(pool[n + q:2 * n].abs().max()) == 0 and int(pool[4 * n - 1024:].abs().max()) == 0   # the refused ones wrote nothing
    # all descriptors fine: status 0
    ok = (C.c_uint64 * 3)(src.data_ptr(), base + 2 * slot, half)
    assert cu.mf_xcopy_debug_probe(ok, 1, base, slot, 4, mapped, bulk) == 0
    torch.cuda.synchronize()
    assert torch.equal(pool[2 * n:2 * n + q], src[:q])


def _prepared_rank(rank, world, url):
    import numpy as np
    import torch
    import memfabric_hybrid as mf
    from memfabric_hybrid import bm
    from memfabric_hybrid_b200.utils import benchutil as bu
    torch.cuda.set_device(0)
    assert mf.initialize() == 0
    cfg = bm.BmConfig()
    cfg.auto_ranking = False
    cfg.rank_id, cfg.start_store = 0, True
    assert bm.initialize(url, 1, 0, cfg) == 0, mf.get_last_err_msg()
    blocks = 4
    nbytes = blocks * bu.KV_BLOCK_BYTES
    pool = (nbytes + (4 << 20)) // (2 << 20) * (2 << 20)
    h = bm.create2(id=0, local_dram_size=0, max_dram_size=0, local_hbm_size=pool, max_hbm_size=pool)
    assert h.join() == 0, mf.get_last_err_msg()
    base = h.peer_rank_ptr(0, bm.BmMemType.DEVICE)
    src = torch.randint(0, 255, (nbytes,), dtype=torch.uint8, device="cuda")
    back = torch.zeros_like(src)
    segs = bu.kv_block_segments(blocks)
    offs = np.array([o for o, _ in segs], dtype=np.uint64)
    sizes = np.array([s for _, s in segs], dtype=np.uint64)
    put = h.create_batch(offs + np.uint64(src.data_ptr()), offs + np.uint64(base), sizes, bm.BmCopyType.L2G)
    get = h.create_batch(offs + np.uint64(base), offs + np.uint64(back.data_ptr()), sizes, bm.BmCopyType.G2L)
    assert put.nbytes == nbytes and get.nbytes == nbytes
    s = torch.cuda.Stream()
    torch.cuda.synchronize()
    # eager: two launches in stream order
    assert put.launch(s.cuda_stream) == 0 and get.launch(s.cuda_stream) == 0, mf.get_last_err_msg()
    s.synchronize()
    eager_ok = bool(torch.equal(back, src))
    # recorded into a CUDA graph and replayed on new data: submission writes nothing on the host
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        assert put.launch(torch.cuda.current_stream().cuda_stream) == 0
        assert get.launch(torch.cuda.current_stream().cuda_stream) == 0
    graph_ok = True
    for seed in (1, 2):
        src.copy_(torch.randint(0, 255, (nbytes,), dtype=torch.uint8, device="cuda", generator=torch.Generator("cuda").manual_seed(seed)))
        back.zero_()
        torch.cuda.synchronize()
        g.replay()
        torch.cuda.synchronize()
        graph_ok = graph_ok and bool(torch.equal(back, src))
    del g
    # a triple outside the pool is refused when the batch is built, host-to-pool types are refused
    bad = None
    try:
        h.create_batch([src.data_ptr()], [base + pool + 4096], [4096], bm.BmCopyType.L2G)
    except RuntimeError as e:
        bad = str(e)
    host = np.zeros(4096, dtype=np.uint8)
    bad2 = None
    try:
        h.create_batch([host.ctypes.data], [base], [4096], bm.BmCopyType.H2G)
    except RuntimeError as e:
        bad2 = str(e)
    mf.get_and_clear_last_err_msg()
    put.destroy()
    get.destroy()
    h.leave()
    h.destroy()
    bm.uninitialize(0)
    mf.uninitialize()
    return eager_ok, graph_ok, bad is not None, bad2 is not None


def test_prepared_batch_launches_and_replays_in_a_cuda_graph():
    """mf_bm_batch_create / _launch: validated once, one launch per submission, capturable."""
    url = f"tcp://127.0.0.1:{free_port()}"
    assert run_ranks(_prepared_rank, 1, (url,), timeout=180) == [(True, True, True, True)]
