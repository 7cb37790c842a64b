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
        torch.cuda._sleep(300_000)  # ~0.15 ms of device idle work: the host gets ahead, so launch latency is not timed
        a.record()
        fn()
        b.record()
        b.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return bu.max_over_ranks(ts[len(ts) // 2])


def collectives(comm, world, flush):
    out = []
    sizes = [1 << 10, 16 << 10, 256 << 10, 1 << 20, 4 << 20, 64 << 20, 256 << 20]
    heap = comm.heap
    mark = heap.mark()
    hx_off, ho_off = heap.alloc(sizes[-1]), heap.alloc(sizes[-1])
    for nbytes in sizes:
        n = nbytes // 2
        x = torch.randn(n, device="cuda").to(torch.bfloat16)
        iters = 20 if nbytes <= (4 << 20) else 6
        fl = flush if nbytes < (128 << 20) else None
        # tensors inside the symmetric heap (what the zbal allocator hands out): peers read and write them in place
        hx, ho = heap.view(hx_off, (n,), torch.bfloat16), heap.view(ho_off, (n,), torch.bfloat16)
        hx.copy_(x)
        ms = _timed(lambda: comm.all_reduce(hx, out=ho, scale=1.0 / world), iters, 3, fl)
        staged = _timed(lambda: comm.all_reduce(x, scale=1.0 / world), iters, 3, fl)
        row = {"op": "allreduce_scaled_bf16", "bytes": nbytes, "us": round(ms * 1e3, 1), "staged_us": round(staged * 1e3, 1),
               "busbw_GBps": round(nbytes * 2 * (world - 1) / max(world, 1) / (ms * 1e-3) / 1e9, 1)}
        if heap.mc_base:
            # "us" went through the NVLink multicast alias (MF_SHM_MULTICAST=1); the same call on peer loads and stores:
            comm.no_multicast = True
            row["peer_ld_st_us"] = round(_timed(lambda: comm.all_reduce(hx, out=ho, scale=1.0 / world), iters, 3, fl) * 1e3, 1)
            comm.no_multicast = False
            row["multicast"] = True
        if world > 1:
            y = x.clone()

            def nccl():
                dist.all_reduce(y)
                y.mul_(1.0 / world)
            row["nccl_us"] = round(_timed(nccl, iters, 3, fl) * 1e3, 1)
        out.append(row)
    # reduce-scatter and all-gather at one large size (fp32 in, bf16 out: the fused cast), heap tensors
    n = (64 << 20) // 4
    hx = heap.view(hx_off, (n,), torch.float32)
    hx.copy_(torch.randn(n, device="cuda"))
    ms = _timed(lambda: comm.reduce_scatter(hx, scale=1.0 / world, out_dtype=torch.bfloat16), 6, 2, flush)
    row = {"op": "reduce_scatter_f32_to_bf16", "bytes": 64 << 20, "us": round(ms * 1e3, 1)}
    if heap.mc_base:
        comm.no_multicast = True
        row["peer_ld_us"] = round(_timed(lambda: comm.reduce_scatter(hx, scale=1.0 / world, out_dtype=torch.bfloat16), 6, 2, flush) * 1e3, 1)
        comm.no_multicast = False
        row["multicast"] = True
    if world > 1:
        y = torch.randn(n, device="cuda")
        o = torch.empty(n // world, device="cuda")

        def nccl_rs():
            dist.reduce_scatter_tensor(o, y)
            o.mul_(1.0 / world).to(torch.bfloat16)
        row["nccl_us"] = round(_timed(nccl_rs, 6, 2, flush) * 1e3, 1)
    out.append(row)
    shard = torch.randn(n // world, device="cuda")
    ho = heap.view(ho_off, (n,), torch.bfloat16)
    ms = _timed(lambda: comm.all_gather(shard, out=ho, out_dtype=torch.bfloat16), 6, 2, flush)
    row = {"op": "all_gather_f32_to_bf16", "bytes": 64 << 20, "us": round(ms * 1e3, 1)}
    if heap.mc_base:
        comm.no_multicast = True
        row["peer_st_us"] = round(_timed(lambda: comm.all_gather(shard, out=ho, out_dtype=torch.bfloat16), 6, 2, flush) * 1e3, 1)
        comm.no_multicast = False
        row["multicast"] = True
    if world > 1:
        g = torch.empty(n, device="cuda")

        def nccl_ag():
            dist.all_gather_into_tensor(g, shard)
            g.to(torch.bfloat16)
        row["nccl_us"] = round(_timed(nccl_ag, 6, 2, flush) * 1e3, 1)
    out.append(row)
    heap.release_to(mark)
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
        extra = {}
        if tokens <= 256:
            # the one-launch low-latency pair on the same routing, replayed as CUDA graphs (the kernels number
            # their calls on the device); y stands in for the caller's expert outputs
            yb = torch.zeros((layer.comm.max_recv, H), dtype=torch.bfloat16, device="cuda")
            ob = torch.empty((tokens, H), dtype=torch.bfloat16, device="cuda")
            idx32, w32 = idx.to(torch.int32).contiguous(), w.to(torch.float32).contiguous()
            for _ in range(2):
                st2 = layer.comm.ll_dispatch(x, idx32, w32)
                layer.comm.ll_combine(yb, st2, out=ob)
            torch.cuda.synchronize()
            bu.barrier()
            mode = "cuda_graph"
            try:
                g1, g2 = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
                with torch.cuda.graph(g1):
                    st2 = layer.comm.ll_dispatch(x, idx32, w32)
                with torch.cuda.graph(g2):
                    layer.comm.ll_combine(yb, st2, out=ob)
                run1, run2 = g1.replay, g2.replay
            except Exception:  # noqa: BLE001  (capture of a cooperative launch refused: time the eager calls)
                torch.cuda.synchronize()
                mode = "eager"
                run1 = lambda: layer.comm.ll_dispatch(x, idx32, w32)
                run2 = lambda: layer.comm.ll_combine(yb, st2, out=ob)
            tl, tcb = [], []
            for it in range(10):
                flush.zero_()
                bu.barrier()
                torch.cuda._sleep(300_000)
                ev[0].record()
                run1()
                ev[1].record()
                torch.cuda._sleep(300_000)
                ev[2].record()
                run2()
                ev[3].record()
                torch.cuda.synchronize()
                if it >= 3:
                    tl.append(ev[0].elapsed_time(ev[1]))
                    tcb.append(ev[2].elapsed_time(ev[3]))
            gemm.check_status()
            extra = {"ll_dispatch_us": round(med(tl) * 1e3, 1), "ll_combine_us": round(med(tcb) * 1e3, 1), "ll_launch": mode}
        res[name] = {**extra, "dispatch_us": round(med(td) * 1e3, 1), "expert_ffn_us": round(f_ms * 1e3, 1), "combine_us": round(med(tc) * 1e3, 1),
                     "recv_rows": rows, "ffn_tflops_fp8": round(flops / (f_ms * 1e-3) / 1e12, 1), "experts": E, "topk": K, "hidden": H}
    return res


def tp_mlp(heap, world, flush):
    from ..models.llama_mlp import TensorParallelMLP
    from ..ops import gemm
    S, H, F = 8192, 8192, 28672
    if world == 1:
        F = 28672 // 8 * 2  # one GPU cannot hold the full layer's work in a short run: use a 1/4-width slice
    mlp = TensorParallelMLP(heap, H, F, S, seed=2, fp8=True)
    x = torch.randn(S // world, H, device="cuda").to(torch.bfloat16)
    ms = _timed(lambda: mlp.forward(x), 6, 3, flush)
    gemm.check_status()
    ms8 = _timed(lambda: mlp.forward_fp8(x), 6, 3, flush)
    gemm.check_status()
    base = _timed(lambda: mlp.forward_baseline(x), 6, 3, flush)
    flops = 2.0 * S * H * (3 * F // world)
    h = mlp.tp.ag_gemm(x, mlp.w_gate_up, swiglu=True)
    ag = _timed(lambda: mlp.tp.ag_gemm(x, mlp.w_gate_up, swiglu=True), 6, 2, flush)
    rs = _timed(lambda: mlp.tp.gemm_rs(h, mlp.w_down), 6, 2, flush)
    gemm.check_status()
    return {"tokens": S, "hidden": H, "ffn": F, "fused_us": round(ms * 1e3, 1), "nccl_cublas_us": round(base * 1e3, 1),
            "fused_tflops_per_gpu": round(flops / (ms * 1e-3) / 1e12, 1), "ag_gemm_swiglu_us": round(ag * 1e3, 1),
            "gemm_rs_us": round(rs * 1e3, 1), "fused_fp8_us": round(ms8 * 1e3, 1),
            "fused_fp8_tflops_per_gpu": round(flops / (ms8 * 1e-3) / 1e12, 1)}


def xcopy_sweep(h, rank, world, flush):
    """KV-block puts / gets of 1-64 blocks, one contiguous 512 MiB copy in both directions, the host legs, and NCCL
    send/recv of the same bytes as the library baseline. Pool copies are enqueued on a stream and timed with events."""
    from ..api import bm
    peer = (rank + 1) % world
    mine, theirs = h.peer_rank_ptr(rank, bm.BmMemType.DEVICE), h.peer_rank_ptr(peer, bm.BmMemType.DEVICE)
    big = 512 << 20
    src = torch.empty(big, dtype=torch.uint8, device="cuda").random_(0, 255)
    dst = torch.empty(big, dtype=torch.uint8, device="cuda")
    side = torch.cuda.Stream()          # the copies and the timing events share this stream
    side.wait_stream(torch.cuda.current_stream())
    stream = side.cuda_stream
    fl = bm.ASYNC_COPY_FLAG | bm.FLAG_USE_EXTERNAL_STREAM
    out = []

    def timed(fn, iters=5):
        with torch.cuda.stream(side):
            return _timed(fn, iters, 2, None)

    for blocks in (1, 8, 64):
        segs = bu.kv_block_segments(blocks)
        nbytes = blocks * bu.KV_BLOCK_BYTES
        put = h.prepare_batch([src.data_ptr() + o for o, _ in segs], [theirs + o for o, _ in segs], [s for _, s in segs])
        get = h.prepare_batch([theirs + o for o, _ in segs], [dst.data_ptr() + o for o, _ in segs], [s for _, s in segs])
        p_ms = timed(lambda: h.copy_prepared(put, bm.BmCopyType.L2G, fl, stream))
        bu.barrier()
        g_ms = timed(lambda: h.copy_prepared(get, bm.BmCopyType.G2L, fl, stream))
        bu.barrier()
        out.append({"op": "kv_blocks", "blocks": blocks, "bytes": nbytes, "put_us": round(p_ms * 1e3, 1), "put_GBps": round(nbytes / p_ms / 1e6, 1),
                    "get_us": round(g_ms * 1e3, 1), "get_GBps": round(nbytes / g_ms / 1e6, 1)})
    # quantising put: bf16 rows become fp8 e4m3 with one factor per 128 elements on their way to the next GPU
    items, per = 1024, 128 * 1024                                   # 1024 pieces of 256 KiB bf16, the size of a KV segment pair
    xb = torch.randn(items * per, dtype=torch.bfloat16, device="cuda")
    q_base, s_base = theirs, theirs + items * per                    # fp8 bytes, then the factors, inside the peer's slice
    side.wait_stream(torch.cuda.current_stream())
    srcs = [xb.data_ptr() + i * per * 2 for i in range(items)]
    dsts = [q_base + i * per for i in range(items)]
    scs = [s_base + i * (per // 128) * 4 for i in range(items)]
    qb = h.prepare_quant_batch(srcs, dsts, [per * 2] * items, scs, 128, fp8=True)
    q_ms = timed(lambda: h.quant_copy_prepared(qb, stream))
    bu.barrier()
    out.append({"op": "quant_put_fp8_1x128", "bytes_in": items * per * 2, "us": round(q_ms * 1e3, 1),
                "in_GBps": round(items * per * 2 / q_ms / 1e6, 1), "wire_GBps": round(items * per * (1 + 4 / 128) / q_ms / 1e6, 1)})
    del xb
    p_ms = timed(lambda: h.copy_data(src.data_ptr(), theirs, big, bm.BmCopyType.L2G, fl, stream))
    bu.barrier()
    g_ms = timed(lambda: h.copy_data(theirs, dst.data_ptr(), big, bm.BmCopyType.G2L, fl, stream))
    bu.barrier()
    row = {"op": "contiguous", "bytes": big, "d2rd_GBps": round(big / p_ms / 1e6, 1), "rd2d_GBps": round(big / g_ms / 1e6, 1)}
    if world > 1:
        prev = (rank - 1) % world

        def nccl():
            ops = [dist.P2POp(dist.isend, src, peer), dist.P2POp(dist.irecv, dst, prev)]
            for r in dist.batch_isend_irecv(ops):
                r.wait()
        row["nccl_send_recv_GBps"] = round(big / timed(nccl) / 1e6, 1)
    out.append(row)
    # host legs: pinned host memory <-> the pool (PCIe)
    host = torch.empty(256 << 20, dtype=torch.uint8).pin_memory()
    n = host.numel()
    h2d = timed(lambda: h.copy_data(host.data_ptr(), mine, n, bm.BmCopyType.H2G, fl, stream))
    d2h = timed(lambda: h.copy_data(mine, host.data_ptr(), n, bm.BmCopyType.G2H, fl, stream))
    row = {"op": "host_legs", "bytes": n, "h2d_GBps": round(n / h2d / 1e6, 1), "d2h_GBps": round(n / d2h / 1e6, 1)}
    if world > 1:
        rh2d = timed(lambda: h.copy_data(host.data_ptr(), theirs, n, bm.BmCopyType.H2G, fl, stream))
        bu.barrier()
        row["h2rd_GBps"] = round(n / rh2d / 1e6, 1)
    out.append(row)
    torch.cuda.synchronize()
    return out


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
    try:
        out["xcopy"] = xcopy_sweep(_bm_handle, rank, world, flush)
    except Exception as e:  # noqa: BLE001
        out["xcopy"] = {"error": repr(e)[:200]}
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
