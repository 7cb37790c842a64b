"""Tiny end-to-end pass on cuda:0 used by ``__graft_entry__.smoke``: a one-rank HBM + DRAM pool, batched
xcopy in every direction a single rank has, bit-exact checks; then the optional kernel groups."""
from __future__ import annotations

import socket


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def run() -> None:
    import torch

    import memfabric_hybrid as mf
    from memfabric_hybrid import bm
    from memfabric_hybrid_b200 import _native

    _native.cuda()  # fail loudly when the CUDA library is missing on a GPU box
    torch.cuda.set_device(0)
    assert mf.initialize() == 0
    cfg = bm.BmConfig()
    cfg.rank_id = 0
    cfg.start_store = True
    assert bm.initialize(f"tcp://127.0.0.1:{_free_port()}", 1, 0, cfg) == 0, mf.get_last_err_msg()
    MiB = 1 << 20
    h = bm.create2(id=0, local_dram_size=16 * MiB, max_dram_size=16 * MiB, local_hbm_size=64 * MiB, max_hbm_size=64 * MiB)
    assert h.join() == 0, mf.get_last_err_msg()
    dev = h.peer_rank_ptr(0, bm.BmMemType.DEVICE)
    hst = h.peer_rank_ptr(0, bm.BmMemType.HOST)
    x = torch.randn(4 * MiB // 2, dtype=torch.bfloat16, device="cuda")
    torch.cuda.synchronize()  # the pool copies on its own stream: x must be complete first
    n, seg = 32, 128 * 1024
    srcs = [x.data_ptr() + i * seg for i in range(n)]
    dsts = [dev + (n - 1 - i) * seg for i in range(n)]  # scattered: reversed order
    assert h.copy_data_batch(srcs, dsts, [seg] * n, n, bm.BmCopyType.L2G, 0) == 0, mf.get_last_err_msg()
    y = torch.empty_like(x)
    assert h.copy_data_batch(dsts, [y.data_ptr() + i * seg for i in range(n)], [seg] * n, n, bm.BmCopyType.G2L, 0) == 0
    torch.cuda.synchronize()
    assert torch.equal(x.view(torch.int16), y.view(torch.int16)), "L2G/G2L round trip differs"
    # device pool -> DRAM pool -> local host
    assert h.copy_data(dev, hst, 4 * MiB, bm.BmCopyType.G2G, 0) == 0, mf.get_last_err_msg()
    out = torch.empty(4 * MiB // 2, dtype=torch.bfloat16)
    assert h.copy_data(hst, out.data_ptr(), 4 * MiB, bm.BmCopyType.GH2H, 0) == 0, mf.get_last_err_msg()
    want = x.view(-1, seg // 2).flip(0).reshape(-1).cpu()
    assert torch.equal(out.view(torch.int16), want.view(torch.int16)), "GD->GH->LH differs"
    stats = h.copy_stats()
    assert stats["kernel_launches"] > 0, f"the SM copy kernel did not run: {stats}"
    h.leave()
    h.destroy()
    bm.uninitialize(0)
    mf.uninitialize()
    try:
        from memfabric_hybrid_b200.ops import smoke_ops
    except ImportError:
        return
    smoke_ops.run()
