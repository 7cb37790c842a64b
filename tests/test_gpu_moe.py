"""MoE expert parallelism: layout, fp8 dispatch, grouped fp8 GEMMs and combine against fp32 references."""
import pytest
import torch

from conftest import free_port
from mp_util import run_ranks

pytestmark = pytest.mark.gpu


def _deq(q, s):
    """fp8 rows [R, K] with 1x128 scales [R, K/128] -> fp32."""
    R, K = q.shape
    return (q.float().view(R, K // 128, 128) * s[:, :, None]).view(R, K)


def _deq_w(q, s):
    *lead, Nn, K = q.shape
    return (q.float().reshape(*lead, Nn // 128, 128, K // 128, 128) * s[..., :, None, :, None]).reshape(*lead, Nn, K)


def test_grouped_gemm_fp8_plain_and_swiglu():
    from memfabric_hybrid_b200.ops import gemm, moe as M
    cu = M._cu()
    torch.manual_seed(0)
    G, N, K = 4, 256, 512
    counts = [130, 0, 7, 300]
    off = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device="cuda")
    R = sum(counts)
    x = torch.randn(R, K, device="cuda").to(torch.bfloat16)
    xq = torch.empty(R, K, dtype=torch.uint8, device="cuda")
    xs = torch.empty(R, K // 128, dtype=torch.float32, device="cuda")
    assert cu.mf_quant_rows_fp8(x.data_ptr(), K, off[G:].data_ptr(), K, xq.data_ptr(), xs.data_ptr(), 64,
                                torch.cuda.current_stream().cuda_stream) == 0
    xd = _deq(xq.view(torch.float8_e4m3fn), xs)
    assert (xd - x.float()).abs().max() <= 0.07 * x.float().abs().max()
    w = (torch.randn(G, N, K, device="cuda") * 0.05).to(torch.bfloat16)
    wq, ws = M.quantize_weight_fp8(w)
    wd = _deq_w(wq, ws)
    out = torch.zeros(R, N, dtype=torch.bfloat16, device="cuda")
    st = gemm.status_word()
    rc = cu.mf_grouped_gemm_fp8(xq.data_ptr(), xs.data_ptr(), R, wq.data_ptr(), ws.data_ptr(), off.data_ptr(), G, N, K, out.data_ptr(), N, 0,
                                None, None, 0, 1, st.data_ptr(), gemm.sm_count(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    gemm.check_status()
    ref = torch.cat([xd[off[g]:off[g + 1]] @ wd[g].t() for g in range(G)])
    assert (out.float() - ref).abs().max() <= 2e-2 * ref.abs().max() + 1e-3
    # SwiGLU: B rows are [gate (N/2) | up (N/2)]; the kernel takes the tile-interleaved copy
    wi = M.interleave_gate_up_fp8(wq, tile=64)   # the 128 x 128 kernel pairs 64 gate rows with 64 up rows
    out2 = torch.zeros(R, N // 2, dtype=torch.bfloat16, device="cuda")
    rc = cu.mf_grouped_gemm_fp8(xq.data_ptr(), xs.data_ptr(), R, wi.data_ptr(), ws.data_ptr(), off.data_ptr(), G, N, K, out2.data_ptr(), N // 2,
                                1, None, None, 0, 1, st.data_ptr(), gemm.sm_count(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    gemm.check_status()
    ref2 = torch.nn.functional.silu(ref[:, :N // 2]) * ref[:, N // 2:]
    assert (out2.float() - ref2).abs().max() <= 3e-2 * ref2.abs().max() + 1e-3


@pytest.mark.parametrize("G,N,K,counts", [(4, 256, 512, [130, 0, 7, 300]), (3, 512, 768, [1, 257, 128]), (2, 1024, 2048, [640, 513])])
def test_grouped_gemm_fp8_block_scaled(G, N, K, counts):
    """The 128 x 256 kernel whose scales are applied by the tensor core (UE8M0 bytes in TMEM): plain, SwiGLU, and
    SwiGLU + re-quantisation epilogues against fp32 references on the dequantised operands. K = 768 has a partial
    group of K blocks (6 = 4 + 2)."""
    from memfabric_hybrid_b200.ops import gemm, moe as M
    cu = M._cu()
    torch.manual_seed(G * N + K)
    s = torch.cuda.current_stream().cuda_stream
    off = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device="cuda")
    R = sum(counts)
    # rows of very different magnitude, so that a wrong scale byte or a wrong row shows
    x = (torch.randn(R, K, device="cuda") * torch.logspace(-2, 2, R, device="cuda")[:, None]).to(torch.bfloat16)
    xq = torch.empty(R, K, dtype=torch.uint8, device="cuda")
    xs = torch.empty(R, K // 128, dtype=torch.float32, device="cuda")
    assert cu.mf_quant_rows_fp8(x.data_ptr(), K, off[G:].data_ptr(), K, xq.data_ptr(), xs.data_ptr(), 64, s) == 0
    assert torch.equal(xs, torch.exp2(torch.round(torch.log2(xs)))), "activation scales must be powers of two"
    xd = _deq(xq.view(torch.float8_e4m3fn), xs)
    w = (torch.randn(G, N, K, device="cuda") * 0.05 * torch.logspace(-1, 1, N // 128, device="cuda").repeat_interleave(128)[None, :, None]).to(torch.bfloat16)
    wq, ws = M.quantize_weight_fp8(w)
    assert torch.equal(ws, torch.exp2(torch.round(torch.log2(ws))))
    wd = _deq_w(wq, ws)
    ref = torch.cat([xd[off[g]:off[g + 1]] @ wd[g].t() for g in range(G)])
    st = gemm.status_word()
    assert cu.mf_grouped_gemm_fp8_mx_supported(G, N, K, 0) == 1
    out = torch.zeros(R, N, dtype=torch.bfloat16, device="cuda")
    assert cu.mf_grouped_gemm_fp8_mx(xq.data_ptr(), xs.data_ptr(), R, wq.data_ptr(), ws.data_ptr(), off.data_ptr(), G, N, K, out.data_ptr(), N, None, 0,
                                     None, None, 0, 1, st.data_ptr(), gemm.sm_count(), s) == 0
    torch.cuda.synchronize()
    gemm.check_status()
    rowmax = ref.abs().amax(dim=1, keepdim=True)
    assert ((out.float() - ref).abs() <= 2e-2 * rowmax + 1e-5).all(), float(((out.float() - ref).abs() / (rowmax + 1e-9)).max())
    # SwiGLU (bf16 out) and SwiGLU + re-quantisation (fp8 + power-of-two scale per 128 outputs)
    wi = M.interleave_gate_up_fp8(wq, tile=128)
    ref2 = torch.nn.functional.silu(ref[:, :N // 2]) * ref[:, N // 2:]
    rowmax2 = ref2.abs().amax(dim=1, keepdim=True)
    out2 = torch.zeros(R, N // 2, dtype=torch.bfloat16, device="cuda")
    assert cu.mf_grouped_gemm_fp8_mx(xq.data_ptr(), xs.data_ptr(), R, wi.data_ptr(), ws.data_ptr(), off.data_ptr(), G, N, K, out2.data_ptr(), N // 2, None,
                                     1, None, None, 0, 1, st.data_ptr(), gemm.sm_count(), s) == 0
    torch.cuda.synchronize()
    gemm.check_status()
    assert ((out2.float() - ref2).abs() <= 3e-2 * rowmax2 + 1e-5).all()
    hq = torch.zeros(R, N // 2, dtype=torch.uint8, device="cuda")
    hs = torch.zeros(R, N // 256, dtype=torch.float32, device="cuda")
    assert cu.mf_grouped_gemm_fp8_mx(xq.data_ptr(), xs.data_ptr(), R, wi.data_ptr(), ws.data_ptr(), off.data_ptr(), G, N, K, hq.data_ptr(), N // 2,
                                     hs.data_ptr(), 3, None, None, 0, 1, st.data_ptr(), gemm.sm_count(), s) == 0
    torch.cuda.synchronize()
    gemm.check_status()
    assert torch.equal(hs, torch.exp2(torch.round(torch.log2(hs))))
    hd = _deq(hq.view(torch.float8_e4m3fn), hs)
    # fp8 e4m3 keeps 3 mantissa bits: each value is within 1/16 of itself plus the block's smallest step
    blockmax = ref2.view(R, N // 256, 128).abs().amax(dim=2, keepdim=True).expand(R, N // 256, 128).reshape(R, N // 2)
    assert ((hd - ref2).abs() <= 0.07 * ref2.abs() + 0.02 * blockmax + 1e-6).all()
    # the same bytes as the stand-alone quantiser produces from the bf16 SwiGLU output of the kernel above
    hq2, hs2 = torch.empty_like(hq), torch.empty_like(hs)
    assert cu.mf_quant_rows_fp8(out2.data_ptr(), N // 2, off[G:].data_ptr(), N // 2, hq2.data_ptr(), hs2.data_ptr(), 64, s) == 0
    torch.cuda.synchronize()
    assert torch.equal(hs, hs2) and torch.equal(hq, hq2)


def _moe_ranks(rank, world, url, T, H, I, E, K, sync):
    import torch
    from memfabric_hybrid_b200.ops import gemm
    from memfabric_hybrid_b200.ops.heap import SymmetricHeap
    from memfabric_hybrid_b200.models.deepseek_moe import ExpertParallelMoE
    from memfabric_hybrid_b200.ops import moe as M
    dev = rank % torch.cuda.device_count()
    max_recv = T * world * min(K, E // world)
    need = (2 << 20) + max_recv * (H + H // 128 * 4 + 16) + T * K * H * 2 + (4 << 20)
    heap = SymmetricHeap(url, world, rank, dev, need)
    layer = ExpertParallelMoE(heap, H, I, E, K, max_tokens=T, seed=5)
    worst = 0.0
    for it in range(2):
        def inputs(r):
            g = torch.Generator("cuda").manual_seed(97 * it + r)
            return (torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16), torch.randn(T, E, device="cuda", generator=g))
        x, logits = inputs(rank)
        y = layer.forward(x, logits)
        torch.cuda.synchronize()
        gemm.check_status()
        # reference: quantise the token like the dispatch does, run every chosen expert in fp32 on dequantised fp8 weights
        idx, w = layer.route(logits, K)
        xq, xs = torch.empty(T, H, dtype=torch.uint8, device="cuda"), torch.empty(T, H // 128, device="cuda")
        n = torch.tensor([T], dtype=torch.int32, device="cuda")
        M._cu().mf_quant_rows_fp8(x.data_ptr(), H, n.data_ptr(), H, xq.data_ptr(), xs.data_ptr(), 64, torch.cuda.current_stream().cuda_stream)
        xd = (xq.view(torch.float8_e4m3fn).float().view(T, H // 128, 128) * xs[:, :, None]).view(T, H)
        ref = torch.zeros(T, H, device="cuda")
        el = E // world
        for r in range(world):
            w1, w2 = layer.make_weights(r, 5, x.device)
            w1q, w1s = M.quantize_weight_fp8(w1)
            w2q, w2s = M.quantize_weight_fp8(w2)
            w1d = (w1q.float().reshape(el, 2 * I // 128, 128, H // 128, 128) * w1s[:, :, None, :, None]).reshape(el, 2 * I, H)
            w2d = (w2q.float().reshape(el, H // 128, 128, I // 128, 128) * w2s[:, :, None, :, None]).reshape(el, H, I)
            for le in range(el):
                e = r * el + le
                tk = (idx == e).nonzero()
                if tk.numel() == 0:
                    continue
                rows = xd[tk[:, 0]]
                gu = rows @ w1d[le].t()
                h = (torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]).to(torch.bfloat16)
                hq, hs = torch.empty(h.shape[0], I, dtype=torch.uint8, device="cuda"), torch.empty(h.shape[0], I // 128, device="cuda")
                nn_ = torch.tensor([h.shape[0]], dtype=torch.int32, device="cuda")
                M._cu().mf_quant_rows_fp8(h.data_ptr(), I, nn_.data_ptr(), I, hq.data_ptr(), hs.data_ptr(), 64,
                                          torch.cuda.current_stream().cuda_stream)
                hd = (hq.view(torch.float8_e4m3fn).float().view(-1, I // 128, 128) * hs[:, :, None]).view(-1, I)
                yrows = (hd @ w2d[le].t()) * w[tk[:, 0], tk[:, 1]][:, None]
                ref.index_add_(0, tk[:, 0], yrows.to(torch.bfloat16).float())
        err = (y.float() - ref).abs().max().item() / (ref.abs().max().item() + 1e-9)
        worst = max(worst, err)
    st = heap.status()[0]
    heap.close()
    SymmetricHeap.shutdown()
    return worst, st


def test_moe_layer_world1():
    url = f"127.0.0.1:{free_port()}"
    (worst, st), = run_ranks(_moe_ranks, 1, (url, 256, 512, 256, 8, 4), timeout=300, with_barrier=True)
    assert st == 0 and worst < 4e-2, (worst, st)


@pytest.mark.multigpu
def test_moe_layer_multi_gpu():
    n = 2 if torch.cuda.device_count() < 4 else 4
    url = f"127.0.0.1:{free_port()}"
    res = run_ranks(_moe_ranks, n, (url, 256, 512, 256, 16, 4), timeout=300, with_barrier=True)
    for worst, st in res:
        assert st == 0 and worst < 4e-2, res


def _canary_rank(rank, world, url, sync):
    import torch
    from memfabric_hybrid_b200.ops import gemm
    from memfabric_hybrid_b200.ops.heap import SymmetricHeap
    from memfabric_hybrid_b200.models.deepseek_moe import ExpertParallelMoE
    T, H, I, E, K = 128, 512, 256, 8, 4
    heap = SymmetricHeap(url, 1, 0, 0, (2 << 20) + T * K * (H + H // 128 * 4 + 16) + T * K * H * 2 + (4 << 20))
    layer = ExpertParallelMoE(heap, H, I, E, K, max_tokens=T, seed=5)
    assert len(layer.comm._guards) == 5
    g = torch.Generator("cuda").manual_seed(1)
    x = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
    logits = torch.randn(T, E, device="cuda", generator=g)
    layer.forward(x, logits)            # checks the guards at the end of combine
    layer.forward(x, logits)
    gemm.check_status()
    # a store that runs past the token rows lands in the guard behind them
    heap.view(layer.comm._guards[1], (4,), torch.int32)[2] = 7
    try:
        layer.comm.check_canaries()
        caught = False
    except RuntimeError as e:
        caught = "guard 1" in str(e)
    heap.close()
    SymmetricHeap.shutdown()
    return caught


def test_moe_receive_areas_are_guarded_by_canaries():
    url = f"127.0.0.1:{free_port()}"
    assert run_ranks(_canary_rank, 1, (url,), timeout=300, with_barrier=True, env={"MF_MOE_CANARY": "1"}) == [True]
