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
