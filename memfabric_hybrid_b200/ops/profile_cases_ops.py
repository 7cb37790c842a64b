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
        ms_ours = _time(lambda: gemm.gemm_bf16(a, b, c, pair=False), args.iters, 3, flush)
        ms_pair = _time(lambda: gemm.gemm_bf16(a, b, c, pair=True), args.iters, 3, flush)
        gemm.check_status()
        ms_lib = _time(lambda: torch.matmul(a, b.t(), out=c), args.iters, 3, flush)
        fl = 2.0 * M * N * K
        out.append({"M": M, "N": N, "K": K, "ours_ms": round(ms_ours, 4), "ours_tflops": round(fl / ms_ours / 1e9, 1),
                    "pair_ms": round(ms_pair, 4), "pair_tflops": round(fl / ms_pair / 1e9, 1),
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
    T, H, I, E, K = (args.tokens, 7168, 2048, 32, 8) if getattr(args, "shape", "small") == "dsv3" else (args.tokens, 2048, 1024, 16, 4)
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


def case_gemm_fp8(args) -> None:
    """Grouped fp8 GEMMs of the DeepSeek-V3 expert FFN (gate/up: N 4096, K 7168; down: N 7168, K 2048) on --tokens rows per
    expert and 8 experts (operands 290 MB / 130 MB: larger than L2): the 128 x 256 kernel with tensor-core block scaling
    (SwiGLU + re-quantisation epilogue, plain epilogue) next to the 128 x 128 kernel that applies the scales in registers.
    A band of rows is checked against an fp32 reference of the dequantised operands."""
    from . import gemm, moe as M
    cu = M._cu()
    s = torch.cuda.current_stream().cuda_stream
    st = gemm.status_word()
    G, per = 8, max(128, args.tokens)
    R = G * per
    off = (torch.arange(0, G + 1, dtype=torch.int32, device="cuda") * per).contiguous()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    gen = torch.Generator("cuda").manual_seed(1)
    out = []
    for name, N, K, epi in (("gate_up_swiglu_requant", 4096, 7168, 3), ("down_plain", 7168, 2048, 0)):
        aq = (torch.randn(R, K, device="cuda", generator=gen) * 4).to(torch.float8_e4m3fn)
        bq = (torch.randn(G, N, K, device="cuda", generator=gen) * 4).to(torch.float8_e4m3fn)
        a_s = torch.exp2(torch.randint(-3, 4, (R, K // 128), device="cuda", generator=gen).float())
        b_s = torch.exp2(torch.randint(-3, 4, (G, N // 128, K // 128), device="cuda", generator=gen).float())
        flops = 2.0 * R * N * K
        if epi == 3:
            bi = M.interleave_gate_up_fp8(bq.view(torch.uint8), 128)
            hq = torch.empty(R, N // 2, dtype=torch.uint8, device="cuda")
            hs = torch.empty(R, N // 256, dtype=torch.float32, device="cuda")
            new = lambda: cu.mf_grouped_gemm_fp8_mx(aq.data_ptr(), a_s.data_ptr(), R, bi.data_ptr(), b_s.data_ptr(), off.data_ptr(), G, N, K, hq.data_ptr(),
                                                    N // 2, hs.data_ptr(), 3, None, None, 0, 1, st.data_ptr(), gemm.sm_count(), s)
        else:
            o_new = torch.empty(R, N, dtype=torch.bfloat16, device="cuda")
            new = lambda: cu.mf_grouped_gemm_fp8_mx(aq.data_ptr(), a_s.data_ptr(), R, bq.data_ptr(), b_s.data_ptr(), off.data_ptr(), G, N, K, o_new.data_ptr(), N,
                                                    None, 0, None, None, 0, 1, st.data_ptr(), gemm.sm_count(), s)
        o_old = torch.empty(R, N, dtype=torch.bfloat16, device="cuda")
        old = lambda: cu.mf_grouped_gemm_fp8(aq.data_ptr(), a_s.data_ptr(), R, bq.data_ptr(), b_s.data_ptr(), off.data_ptr(), G, N, K, o_old.data_ptr(), N, 0,
                                             None, None, 0, 1, st.data_ptr(), gemm.sm_count(), s)
        assert new() == 0 and old() == 0
        torch.cuda.synchronize()
        gemm.check_status()
        # reference on the first 64 rows of the last expert
        r0 = (G - 1) * per
        ad = (aq[r0:r0 + 64].float().view(64, K // 128, 128) * a_s[r0:r0 + 64, :, None]).view(64, K)
        bd = (bq[G - 1].float().view(N // 128, 128, K // 128, 128) * b_s[G - 1][:, None, :, None]).view(N, K)
        ref = ad @ bd.t()
        if epi == 3:
            ref = torch.nn.functional.silu(ref[:, :N // 2]) * ref[:, N // 2:]
            got = (hq[r0:r0 + 64].view(torch.float8_e4m3fn).float().view(64, N // 256, 128) * hs[r0:r0 + 64, :, None]).view(64, N // 2)
            tol = 0.08
        else:
            got = o_new[r0:r0 + 64].float()
            tol = 0.02
        rm = ref.abs().amax(dim=1, keepdim=True)
        assert ((got - ref).abs() <= tol * rm + 1e-3).all(), float(((got - ref).abs() / (rm + 1e-9)).max())
        ms_new = _time(new, args.iters, 2, flush)
        ms_old = _time(old, args.iters, 2, flush)
        gemm.check_status()
        out.append({"gemm": name, "rows": R, "N": N, "K": K, "block_scaled_ms": round(ms_new, 4), "block_scaled_tflops": round(flops / ms_new / 1e9, 1),
                    "scales_in_registers_ms": round(ms_old, 4), "scales_in_registers_tflops": round(flops / ms_old / 1e9, 1)})
    print(json.dumps({"case": "gemm_fp8", "results": out}))
