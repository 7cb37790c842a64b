"""Profiler / timing cases of the kernel families in ``ops`` (run through ``utils.profile_cases``)."""
from __future__ import annotations

import json

import torch


def _time(fn, iters=10, warmup=3, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2 * iters)]
    for i in range(iters):
        if flush is not None:
            flush.zero_()  # a write larger than L2 between timed iterations
        ev[2 * i].record()
        fn()
        ev[2 * i + 1].record()
    torch.cuda.synchronize()
    ts = sorted(ev[2 * i].elapsed_time(ev[2 * i + 1]) for i in range(iters))
    return ts[len(ts) // 2]


def case_gemm(args) -> None:
    """bf16 GEMM throughput of the tcgen05 kernel next to cuBLAS (torch.matmul) on the same shapes."""
    from . import gemm
    shapes = [(8192, 8192, 8192), (8192, 7168, 8192), (8192, 8192, 3584), (4096, 4096, 7168)]
    if args.size_mb <= 64:  # small capture case
        shapes = [(2048, 2048, 2048)]
    elif args.size_mb <= 128:  # capture case whose operands (148 MB) exceed L2
        shapes = [(4096, 4096, 7168)]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    out = []
    for M, N, K in shapes:
        a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        b = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
        c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        ms_ours = _time(lambda: gemm.gemm_bf16(a, b, c), args.iters, 3, flush)
        gemm.check_status()
        ms_lib = _time(lambda: torch.matmul(a, b.t(), out=c), args.iters, 3, flush)
        fl = 2.0 * M * N * K
        out.append({"M": M, "N": N, "K": K, "ours_ms": round(ms_ours, 4), "ours_tflops": round(fl / ms_ours / 1e9, 1),
                    "cublas_ms": round(ms_lib, 4), "cublas_tflops": round(fl / ms_lib / 1e9, 1)})
    print(json.dumps({"case": "gemm_bf16", "results": out}))


def case_allreduce(args) -> None:
    """Two-shot all-reduce of 8 emulated ranks in one cooperative launch (rank = blockIdx.y): the data path of
    the multi-GPU kernel with every "peer" on this GPU. --size-mb is the per-rank payload."""
    from .collectives import Communicator
    from .heap import EmulatedHeap
    world = 8
    n = (args.size_mb << 20) // 2
    stage = (n * 2 + 4095) // 4096 * 4096
    heap = EmulatedHeap(world, (1 << 20) + 4 * stage + (1 << 20))
    c = Communicator(heap, stage_bytes=stage)
    x = torch.randn(world, n, device="cuda").to(torch.bfloat16)
    out = torch.empty_like(x)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    ms = _time(lambda: c.all_reduce(x, out=out, scale=1.0 / world, algo="twoshot"), args.iters, 2, flush)
    ref = x.float().sum(0) / world
    torch.testing.assert_close(out[3].float(), ref, rtol=3e-2, atol=3e-2)
    assert heap.status()[0] == 0
    # per emulated rank: stage copy (read n, write n), reduce (read n from 8 slots, write n/8 x 8), copy out (read n, write n)
    traffic = world * n * 2 * 6
    print(json.dumps({"case": "allreduce_twoshot_emulated_8", "bytes_per_rank": n * 2, "ms": round(ms, 4),
                      "device_traffic_GBps": round(traffic / ms / 1e6, 1)}))


def _moe_single(tokens: int, hidden: int, inter: int, experts: int, topk: int):
    import socket
    from ..models.deepseek_moe import ExpertParallelMoE
    from .heap import SymmetricHeap
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    heap = SymmetricHeap(f"127.0.0.1:{port}", 1, 0, 0, 3 << 30)
    layer = ExpertParallelMoE(heap, hidden, inter, experts, topk, max_tokens=tokens, max_recv=tokens * topk, seed=1)
    g = torch.Generator("cuda").manual_seed(0)
    x = torch.randn(tokens, hidden, device="cuda", generator=g).to(torch.bfloat16)
    idx, w = layer.route(torch.randn(tokens, experts, device="cuda", generator=g), topk)
    return heap, layer, x, idx, w


def case_moe(args) -> None:
    """One rank owning all experts: layout + notify + fused fp8 dispatch, grouped fp8 GEMMs (SwiGLU; down +
    combine push), slot reduce; checked against an fp32 reference of the same quantised computation."""
    from . import gemm
    from .heap import SymmetricHeap
    T, H, I, E, K = args.tokens, 2048, 1024, 16, 4
    heap, layer, x, idx, w = _moe_single(T, H, I, E, K)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    td, tf, tc = [], [], []
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    for it in range(args.iters + 2):
        flush.zero_()
        ev[0].record()
        st = layer.comm.dispatch(x, idx, w)
        ev[1].record()
        layer.comm.expert_ffn(st, layer.w1q, layer.w1s, layer.w2q, layer.w2s)
        ev[2].record()
        y = layer.comm.combine(st)
        ev[3].record()
        torch.cuda.synchronize()
        if it >= 2:
            td.append(ev[0].elapsed_time(ev[1]))
            tf.append(ev[1].elapsed_time(ev[2]))
            tc.append(ev[2].elapsed_time(ev[3]))
    gemm.check_status()
    ref = layer.reference(x, idx, w) if hasattr(layer, "reference") else None
    if ref is not None:
        err = (y.float() - ref.float()).abs().max().item() / max(1e-6, ref.float().abs().max().item())
        assert err < 0.08, f"relative error {err}"
    rows = int(st.row_off[-1].item())
    med = lambda v: sorted(v)[len(v) // 2]
    print(json.dumps({"case": "moe_single_rank", "tokens": T, "rows": rows, "dispatch_ms": round(med(td), 4), "ffn_ms": round(med(tf), 4),
                      "combine_ms": round(med(tc), 4), "ffn_tflops_fp8": round(2.0 * rows * 3 * I * H / med(tf) / 1e9, 1)}))
    torch.cuda.synchronize()
    heap.close()
    SymmetricHeap.shutdown()
