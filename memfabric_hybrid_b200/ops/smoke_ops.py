"""Second half of the smoke pass: the kernel families on tiny shapes, each checked against PyTorch.
  * tcgen05 bf16 GEMM (plain and SwiGLU epilogue)
  * collectives with four emulated ranks in one cooperative launch
  * the MoE layer on one rank: fused fp8 dispatch, grouped fp8 GEMMs, combine; and the low-latency pair
"""
from __future__ import annotations

import socket

import torch


def run() -> None:
    from . import gemm
    from .collectives import Communicator
    from .heap import EmulatedHeap, SymmetricHeap
    from ..models.deepseek_moe import ExpertParallelMoE

    torch.manual_seed(0)
    a = torch.randn(256, 512, device="cuda").to(torch.bfloat16)
    b = (torch.randn(384, 512, device="cuda") * 0.05).to(torch.bfloat16)
    c = gemm.gemm_bf16(a, b)
    gemm.check_status()
    torch.testing.assert_close(c.float(), a.float() @ b.float().t(), rtol=3e-2, atol=3e-2)

    heap = EmulatedHeap(4, (1 << 20) + 4 * (1 << 20) + (1 << 20))
    comm = Communicator(heap, stage_bytes=1 << 20)
    x = torch.randn(4, 50_000, device="cuda")
    out = comm.all_reduce(x, scale=0.25, out_dtype=torch.bfloat16)
    torch.cuda.synchronize()
    torch.testing.assert_close(out[2].float(), x.sum(0) / 4, rtol=2e-2, atol=2e-2)
    assert heap.status()[0] == 0, f"a device wait gave up: {heap.status()}"

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    sheap = SymmetricHeap(f"127.0.0.1:{port}", 1, 0, 0, 256 << 20)
    T, H, I, E, K = 64, 1024, 512, 8, 2
    layer = ExpertParallelMoE(sheap, H, I, E, K, max_tokens=T, max_recv=T * K, seed=3)
    xt = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    logits = torch.randn(T, E, device="cuda")
    y = layer.forward(xt, logits)
    # fp32 reference from the bf16 master weights (the fp8 path differs by quantisation noise only)
    idx, w = layer.route(logits, K)
    ref = torch.zeros(T, H, device="cuda")
    for t in range(T):
        for k in range(K):
            e = int(idx[t, k])
            h = layer.w1[e].float() @ xt[t].float()
            act = torch.nn.functional.silu(h[:I]) * h[I:]
            ref[t] += w[t, k] * (layer.w2[e].float() @ act)
    torch.cuda.synchronize()
    gemm.check_status()
    err = (y.float() - ref).abs().max().item() / max(ref.abs().max().item(), 1e-6)
    assert err < 0.1, f"MoE layer differs from the fp32 reference: relative error {err}"
    # low-latency pair with identity experts: the output is x times the sum of the routing weights (= 1)
    st = layer.comm.ll_dispatch(xt, idx, w)
    n = int(st.row_off[-1].item())
    q, sc = layer.comm.recv_x()[:n], layer.comm.recv_scale()[:n]
    rows = (q.float().view(n, H // 128, 128) * sc.view(n, H // 128, 1)).view(n, H).to(torch.bfloat16)
    back = layer.comm.ll_combine(rows, st)
    torch.cuda.synchronize()
    gemm.check_status()
    torch.testing.assert_close(back.float(), xt.float(), rtol=0.08, atol=0.08)
    sheap.close()
    SymmetricHeap.shutdown()
