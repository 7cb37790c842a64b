"""Secondary measurements printed in bench.py's JSON line under "extras": the collective sweep against
NCCL, the DeepSeek-V3-shaped MoE layer (dispatch / expert FFN / combine, prefill and 128-token decode) and
the Llama-3-70B-shaped tensor-parallel MLP against NCCL + cuBLAS. Everything is timed on the device with
CUDA events (median of the timed iterations, max over ranks) after warm-up; buffers are larger than L2 or
an L2-sized buffer is rewritten between iterations."""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from . import benchutil as bu


def _timed(fn, iters, warmup, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return bu.max_over_ranks(ts[len(ts) // 2])


def collectives(comm, world, flush):
    out = []
    sizes = [1 << 10, 16 << 10, 256 << 10, 4 << 20, 64 << 20, 256 << 20]
    for nbytes in sizes:
        n = nbytes // 2
        x = torch.randn(n, device="cuda").to(torch.bfloat16)
        iters = 20 if nbytes <= (4 << 20) else 6
        fl = flush if nbytes < (128 << 20) else None
        ms = _timed(lambda: comm.all_reduce(x, scale=1.0 / world), iters, 3, fl)
        row = {"op": "allreduce_scaled_bf16", "bytes": nbytes, "us": round(ms * 1e3, 1),
               "busbw_GBps": round(nbytes * 2 * (world - 1) / max(world, 1) / (ms * 1e-3) / 1e9, 1)}
        if world > 1:
            y = x.clone()

            def nccl():
                dist.all_reduce(y)
                y.mul_(1.0 / world)
            row["nccl_us"] = round(_timed(nccl, iters, 3, fl) * 1e3, 1)
        out.append(row)
    # reduce-scatter and all-gather at one large size (fp32 in, bf16 out: the fused cast)
    n = (64 << 20) // 4
    x = torch.randn(n, device="cuda")
    ms = _timed(lambda: comm.reduce_scatter(x, scale=1.0 / world, out_dtype=torch.bfloat16), 6, 2, flush)
    out.append({"op": "reduce_scatter_f32_to_bf16", "bytes": 64 << 20, "us": round(ms * 1e3, 1)})
    shard = torch.randn(n // world, device="cuda")
    ms = _timed(lambda: comm.all_gather(shard, out_dtype=torch.bfloat16), 6, 2, flush)
    out.append({"op": "all_gather_f32_to_bf16", "bytes": 64 << 20, "us": round(ms * 1e3, 1)})
    return out


def moe(heap, world, rank, flush):
    from ..models.deepseek_moe import ExpertParallelMoE
    from ..ops import gemm
    res = {}
    H, I, K = 7168, 2048, 8
    E = 32 * world
    T = 4096
    layer = ExpertParallelMoE(heap, H, I, E, K, max_tokens=T, max_recv=int(T * K * 1.3), seed=1)  # balanced routing sends ~T*K rows here; 30 % head-room
    for name, tokens in (("prefill_4096", T), ("decode_128", 128)):
        g = torch.Generator("cuda").manual_seed(rank)
        x = torch.randn(tokens, H, device="cuda", generator=g).to(torch.bfloat16)
        logits = torch.randn(tokens, E, device="cuda", generator=g)
        idx, w = layer.route(logits, K)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        td, tf, tc = [], [], []
        for it in range(6):
            flush.zero_()
            bu.barrier()
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
        med = lambda v: bu.max_over_ranks(sorted(v)[len(v) // 2])
        rows = int(st.row_off[-1].item())
        flops = 2.0 * rows * (2 * I * H + H * I)
        f_ms = med(tf)
        res[name] = {"dispatch_us": round(med(td) * 1e3, 1), "expert_ffn_us": round(f_ms * 1e3, 1), "combine_us": round(med(tc) * 1e3, 1),
                     "recv_rows": rows, "ffn_tflops_fp8": round(flops / (f_ms * 1e-3) / 1e12, 1), "experts": E, "topk": K, "hidden": H}
    return res


def tp_mlp(heap, world, flush):
    from ..models.llama_mlp import TensorParallelMLP
    from ..ops import gemm
    S, H, F = 8192, 8192, 28672
    if world == 1:
        F = 28672 // 8 * 2  # one GPU cannot hold the full layer's work in a short run: use a 1/4-width slice
    mlp = TensorParallelMLP(heap, H, F, S, seed=2)
    x = torch.randn(S // world, H, device="cuda").to(torch.bfloat16)
    ms = _timed(lambda: mlp.forward(x), 6, 3, flush)
    gemm.check_status()
    base = _timed(lambda: mlp.forward_baseline(x), 6, 3, flush)
    flops = 2.0 * S * H * (3 * F // world)
    h = mlp.tp.ag_gemm(x, mlp.w_gate_up, swiglu=True)
    ag = _timed(lambda: mlp.tp.ag_gemm(x, mlp.w_gate_up, swiglu=True), 6, 2, flush)
    rs = _timed(lambda: mlp.tp.gemm_rs(h, mlp.w_down), 6, 2, flush)
    gemm.check_status()
    return {"tokens": S, "hidden": H, "ffn": F, "fused_us": round(ms * 1e3, 1), "nccl_cublas_us": round(base * 1e3, 1),
            "fused_tflops_per_gpu": round(flops / (ms * 1e-3) / 1e12, 1), "ag_gemm_swiglu_us": round(ag * 1e3, 1),
            "gemm_rs_us": round(rs * 1e3, 1)}


def run(rank, world, local, _bm_handle):
    from ..ops.collectives import Communicator
    from ..ops.heap import SymmetricHeap
    addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
    port = int(os.environ.get("MASTER_PORT", "29500")) + 41
    if world == 1:
        import socket
        s = socket.socket()
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
        s.close()
    heap = SymmetricHeap(f"{addr}:{port}", world, rank, local, 7 << 30)
    flush = torch.empty(192 << 20, dtype=torch.uint8, device="cuda")
    out = {}
    comm = Communicator(heap, stage_bytes=64 << 20)
    out["collectives"] = collectives(comm, world, flush)
    mark = heap.mark()
    out["tp_mlp_bf16"] = tp_mlp(heap, world, flush)
    heap.release_to(mark)
    out["moe_ep"] = moe(heap, world, rank, flush)
    st = heap.status()
    out["device_wait_status"] = st[0]
    torch.cuda.synchronize()
    heap.close()
    SymmetricHeap.shutdown()
    return out
