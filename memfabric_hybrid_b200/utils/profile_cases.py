"""Small, self-ending workloads for profiler captures, one per kernel family.

    python -m memfabric_hybrid_b200.utils.profile_cases xcopy [--blocks 16] [--iters 3]

Each case holds well under a few GB on the device, launches the kernel of interest a handful of
times after a short warm-up, checks its result and exits 0.
"""
from __future__ import annotations

import argparse
import socket
import sys


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def case_xcopy(args) -> None:
    import torch

    import memfabric_hybrid as mf
    from memfabric_hybrid import bm
    from memfabric_hybrid_b200.utils import benchutil as bu
    torch.cuda.set_device(0)
    mf.initialize()
    cfg = bm.BmConfig()
    cfg.rank_id = 0
    cfg.start_store = True
    assert bm.initialize(f"tcp://127.0.0.1:{_free_port()}", 1, 0, cfg) == 0, mf.get_last_err_msg()
    step = args.blocks * bu.KV_BLOCK_BYTES
    pool = (step + (4 << 20)) // (2 << 20) * (2 << 20)
    h = bm.create2(id=0, local_dram_size=0, max_dram_size=0, local_hbm_size=pool, max_hbm_size=pool)
    assert h.join() == 0, mf.get_last_err_msg()
    base = h.peer_rank_ptr(0, bm.BmMemType.DEVICE)
    src = torch.randn(step // 2, dtype=torch.bfloat16, device="cuda")
    segs = bu.kv_block_segments(args.blocks)
    batch = h.prepare_batch([src.data_ptr() + o for o, _ in segs], [base + o for o, _ in segs], [s for _, s in segs])
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    for i in range(args.iters + 1):
        if i == 1:
            ev[0].record()
        assert h.copy_prepared(batch, bm.BmCopyType.L2G, 0) == 0, mf.get_last_err_msg()
    ev[1].record()
    torch.cuda.synchronize()
    out = torch.empty_like(src)
    assert h.copy_data(base, out.data_ptr(), step, bm.BmCopyType.G2L, 0) == 0
    assert torch.equal(out.view(torch.int16), src.view(torch.int16))
    ms = ev[0].elapsed_time(ev[1]) / args.iters
    print(f"xcopy {args.blocks} blocks: {ms:.3f} ms per put (incl. host submit + sync), {2 * step / ms / 1e6:.1f} GB/s read+write")
    h.leave()
    h.destroy()
    bm.uninitialize(0)
    mf.uninitialize()


def case_quant(args) -> None:
    """Quantising copy (bf16 -> fp8 e4m3 + 1 x 128 factors) of --size-mb MiB of input into this rank's own slice."""
    import torch

    import memfabric_hybrid as mf
    from memfabric_hybrid import bm
    torch.cuda.set_device(0)
    mf.initialize()
    cfg = bm.BmConfig()
    cfg.rank_id = 0
    cfg.start_store = True
    assert bm.initialize(f"tcp://127.0.0.1:{_free_port()}", 1, 0, cfg) == 0, mf.get_last_err_msg()
    nbytes = args.size_mb << 20
    elems = nbytes // 2
    pool = (elems + elems // 32 + (4 << 20)) // (2 << 20) * (2 << 20)
    h = bm.create2(id=0, local_dram_size=0, max_dram_size=0, local_hbm_size=pool, max_hbm_size=pool)
    assert h.join() == 0, mf.get_last_err_msg()
    base = h.peer_rank_ptr(0, bm.BmMemType.DEVICE)
    x = torch.randn(elems, dtype=torch.bfloat16, device="cuda")
    per = 128 * 1024
    items = elems // per
    qb = h.prepare_quant_batch([x.data_ptr() + i * per * 2 for i in range(items)], [base + i * per for i in range(items)], [per * 2] * items,
                               [base + elems + i * (per // 128) * 4 for i in range(items)], 128, fp8=True)
    s = torch.cuda.current_stream()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    torch.cuda.synchronize()
    for i in range(args.iters + 1):
        if i == 1:
            ev[0].record()
        assert h.quant_copy_prepared(qb, s.cuda_stream) == 0, mf.get_last_err_msg()
    ev[1].record()
    torch.cuda.synchronize()
    q = torch.empty(elems, dtype=torch.uint8, device="cuda")
    f = torch.empty(elems // 128, dtype=torch.float32, device="cuda")
    assert h.copy_data(base, q.data_ptr(), elems, bm.BmCopyType.G2L, 0) == 0
    assert h.copy_data(base + elems, f.data_ptr(), elems // 32, bm.BmCopyType.G2L, 0) == 0
    back = q.view(torch.float8_e4m3fn).float().view(-1, 128) * f[:, None]
    err = float((back - x.float().view(-1, 128)).abs().max())
    assert err <= float(x.float().abs().max()) * 0.07, err
    ms = ev[0].elapsed_time(ev[1]) / args.iters
    print(f"quant {args.size_mb} MiB bf16 -> fp8: {ms * 1e3:.1f} us per call, {nbytes / ms / 1e6:.1f} GB/s of input, "
          f"{(nbytes + elems + elems // 32) / ms / 1e6:.1f} GB/s read+write")
    h.leave()
    h.destroy()
    bm.uninitialize(0)
    mf.uninitialize()


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("case")
    ap.add_argument("--blocks", type=int, default=16)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--tokens", type=int, default=512)
    ap.add_argument("--size-mb", type=int, default=256)
    ap.add_argument("--shape", default="small", choices=["small", "dsv3"], help="moe: 2048/1024/16 experts/top-4, or the DeepSeek-V3 layer")
    args, _ = ap.parse_known_args()
    fn = globals().get("case_" + args.case)
    if fn is None:
        try:
            from memfabric_hybrid_b200.ops import profile_cases_ops
            fn = getattr(profile_cases_ops, "case_" + args.case, None)
        except ImportError:
            fn = None
    if fn is None:
        print(f"unknown case {args.case}", file=sys.stderr)
        return 2
    fn(args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
