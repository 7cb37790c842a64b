"""An HBM pool on one GPU, copies enqueued on the caller's CUDA stream and completed with ``wait``
(examples/memory_pool/01_basic/03 and 06_single_card_external_stream of the reference). Needs a GPU.

    python examples/memory_pool/03_hbm_pool_external_stream.py
"""
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
import _launch  # noqa: E402

MiB = 1 << 20


def main(rank: int, world: int, url: str) -> str:
    import memfabric_hybrid as mf
    from memfabric_hybrid import bm
    torch.cuda.set_device(0)
    torch.zeros(1, device="cuda")
    assert mf.initialize() == 0
    cfg = bm.BmConfig()
    cfg.rank_id, cfg.start_store = rank, True
    assert bm.initialize(url, world, 0, cfg) == 0, mf.get_last_err_msg()
    h = bm.create(id=0, local_dram_size=0, local_hbm_size=256 * MiB, data_op_type=bm.BmDataOpType.SDMA)
    assert h.join() == 0
    base = h.peer_rank_ptr(rank, bm.BmMemType.DEVICE)
    x = torch.arange(4 * MiB, device="cuda", dtype=torch.float32)
    y = torch.zeros_like(x)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    n = x.numel() * 4
    SMEM_BM_FLAG_USE_EXTERNAL_STREAM = bm.ASYNC_COPY_FLAG | bm.FLAG_USE_EXTERNAL_STREAM   # enqueue on our stream, return at once
    assert h.copy_data(x.data_ptr(), base, n, bm.BmCopyType.L2G, SMEM_BM_FLAG_USE_EXTERNAL_STREAM, s.cuda_stream) == 0
    assert h.copy_data(base, y.data_ptr(), n, bm.BmCopyType.G2L, SMEM_BM_FLAG_USE_EXTERNAL_STREAM, s.cuda_stream) == 0
    s.synchronize()
    h.wait()
    ok = bool(torch.equal(x, y))
    h.leave()
    h.destroy()
    bm.uninitialize()
    mf.uninitialize()
    return "ok" if ok else "mismatch"


if __name__ == "__main__":
    res = _launch.run(main, 1, f"tcp://127.0.0.1:{_launch.free_port()}")
    print(res)
    sys.exit(0 if res == ["ok"] else 1)
