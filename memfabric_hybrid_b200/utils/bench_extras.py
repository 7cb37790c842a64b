"""Secondary measurements printed in bench.py's JSON line under "extras": the xcopy sweep of the public API, the
collective grid against NCCL, the DeepSeek-V3-shaped MoE layer (dispatch / expert FFN / combine, prefill and 128-token
decode) against an NCCL all-to-all + library grouped-GEMM layer, and the Llama-3-70B-shaped tensor-parallel MLP (bf16 and
fp8) against NCCL + cuBLAS. Everything is timed on the device with CUDA events (median of the timed iterations, max over
ranks) after warm-up; buffers are larger than L2 or an L2-sized buffer is rewritten between iterations. Before an
operation is timed its result is compared once with NCCL / a PyTorch reference on the same inputs ("verified"), and
every row carries the fraction of its roofline: bytes that must cross NVLink over the measured 770 GB/s per direction
per GPU, or FLOPs over the measured cuBLAS bf16 peak (MEASURED_PEAKS.json when present)."""
from __future__ import annotations

import json
import os
import time

import torch
import torch.distributed as dist

from . import benchutil as bu

NVLINK_GBS = 770.0  # measured peer copy per direction per GPU on this pool (nominal 900)


def _peaks() -> dict:
    for cand in (os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json"),):
        try:
            with open(cand) as f:
                d = json.load(f)
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
        except (OSError, ValueError, KeyError):
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


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


def _all_ranks(ok: bool) -> bool:
    """True when the check held on every rank."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return bool(ok)
    t = torch.tensor([1 if ok else 0], dtype=torch.int32, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return bool(t.item())


def _close(got: torch.Tensor, want: torch.Tensor, rel: float) -> bool:
    g, w = got.float(), want.float()
    return bool(((g - w).abs().max() <= rel * w.abs().max() + 1e-6).item())


def collectives(comm, world, flush, max_bytes=1 << 30):
    """all-reduce (+ fused 1/N scale), reduce-scatter and all-gather, bf16 and fp32, 1 KiB - 1 GiB in powers of two, tensors
    inside the symmetric heap (what the zbal allocator hands out: peers read and write them in place). "us" is what the
    library's selector runs; when the heap has an NVLink multicast alias, "peer_us" and "mc_us" are the same call forced onto
    plain peer loads / stores and onto the multicast alias; "nccl_us" torch.distributed NCCL on the same bytes (with the
    separate scale kernel that the fused epilogue replaces)."""
    out = []
    heap = comm.heap
    mark = heap.mark()
    hx_off, ho_off = heap.alloc(max_bytes, 1024), heap.alloc(max_bytes, 1024)
    sizes = [1 << p for p in range(10, 31) if (1 << p) <= max_bytes]
    mc = bool(heap.mc_base)
    for dtype, dname in ((torch.bfloat16, "bf16"), (torch.float32, "fp32")):
        es = 2 if dtype == torch.bfloat16 else 4
        tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
        src = torch.randn(max_bytes // es, device="cuda", dtype=torch.float32 if es == 4 else torch.bfloat16) if world > 1 else None
        for nbytes in sizes:
            n = nbytes // es
            n -= n % (8 * world)
            if n == 0:
                continue
            iters = 12 if nbytes <= (4 << 20) else (6 if nbytes <= (128 << 20) else 4)
            fl = flush if nbytes < (128 << 20) else None
            hx, ho = heap.view(hx_off, (n,), dtype), heap.view(ho_off, (n,), dtype)
            if src is not None:
                hx.copy_(src[:n])
            else:
                hx.normal_()
            wire = nbytes * (world - 1) / max(world, 1)
            for op in ("allreduce_scaled", "reduce_scatter", "all_gather"):
                m = n // world
                if op == "allreduce_scaled":
                    ours = lambda: comm.all_reduce(hx, out=ho, scale=1.0 / world)
                    floor_us = 2 * wire / NVLINK_GBS / 1e3
                elif op == "reduce_scatter":
                    ours = lambda: comm.reduce_scatter(hx, out=ho[:m], scale=1.0 / world)
                    floor_us = wire / NVLINK_GBS / 1e3
                else:
                    ours = lambda: comm.all_gather(hx[:m], out=ho)
                    floor_us = wire / NVLINK_GBS / 1e3
                row = {"op": f"{op}_{dname}", "bytes": n * es}
                nccl = None
                if world > 1:
                    y = hx.clone()
                    if op == "allreduce_scaled":
                        yo = y

                        def nccl():
                            dist.all_reduce(yo)
                            yo.mul_(1.0 / world)
                    elif op == "reduce_scatter":
                        yo = torch.empty(m, dtype=dtype, device="cuda")

                        def nccl():
                            dist.reduce_scatter_tensor(yo, y)
                            yo.mul_(1.0 / world)
                    else:
                        yo = torch.empty(n, dtype=dtype, device="cuda")

                        def nccl():
                            dist.all_gather_into_tensor(yo, y[:m])
                    # one checked call of each before anything is timed (NCCL works on a copy: its all-reduce is in place)
                    ours()
                    nccl()
                    torch.cuda.synchronize()
                    got = ho[:m] if op == "reduce_scatter" else ho
                    row["verified"] = _all_ranks(_close(got, yo, tol))
                    if op == "allreduce_scaled":
                        y.copy_(hx)
                else:
                    ours()
                    torch.cuda.synchronize()
                    want = hx if op != "reduce_scatter" else hx[:m]
                    row["verified"] = _close(ho[:m] if op == "reduce_scatter" else ho, want, tol)
                us = _timed(ours, iters, 2, fl) * 1e3
                row["us"] = round(us, 1)
                if mc and nbytes > (256 << 10):
                    # both variants forced, next to what the library's selector chose ("us")
                    comm.multicast = False
                    row["peer_us"] = round(_timed(ours, iters, 2, fl) * 1e3, 1)
                    comm.multicast = True
                    row["mc_us"] = round(_timed(ours, iters, 2, fl) * 1e3, 1)
                    comm.multicast = None
                if nccl is not None:
                    row["nccl_us"] = round(_timed(nccl, iters, 2, fl) * 1e3, 1)
                    best = row["us"]
                    row["vs_nccl"] = round(row["nccl_us"] / best, 3)
                    row["roofline_frac"] = round(floor_us / best, 3)
                    if op == "allreduce_scaled":
                        row["busbw_GBps"] = round(2 * wire / (best * 1e-6) / 1e9, 1)
                out.append(row)
        del src
    heap.release_to(mark)
    return out


def alltoallv(heap, world, rank, flush):
    """all-to-all-v of bf16 rows, 16 / 128 MiB of input per rank (the size of the reference's published All2Allv table), even
    splits and splits skewed 3 : 1 towards the next rank, against torch.distributed all_to_all_single (NCCL) on the same splits.
    Checked against NCCL's output before timing."""
    from ..ops.collectives import Communicator
    import torch.distributed as dist
    out = []
    if world < 2:
        return out
    mark = heap.mark()
    comm = Communicator(heap, stage_bytes=(128 << 20) + (1 << 20))
    for nbytes in (16 << 20, 128 << 20):
        n = nbytes // 2
        for skew in (False, True):
            weights = [3.0 if (skew and p == (rank + 1) % world) else 1.0 for p in range(world)]
            unit = 64   # elements: pieces stay 128-byte aligned
            send = [int(n * w / sum(weights)) // unit * unit for w in weights]
            # what every peer sends to me: the same rule seen from its side
            recv = []
            for p in range(world):
                wp = [3.0 if (skew and q == (p + 1) % world) else 1.0 for q in range(world)]
                recv.append(int(n * wp[rank] / sum(wp)) // unit * unit)
            soff = [sum(send[:i]) for i in range(world)]
            roff = [sum(recv[:i]) for i in range(world)]
            x = torch.randn(sum(send), device="cuda").to(torch.bfloat16)
            y = torch.empty(sum(recv), device="cuda", dtype=torch.bfloat16)
            yn = torch.empty_like(y)
            ours = lambda: comm.all_to_all_v(x, y, send, soff, recv, roff)
            nccl = lambda: dist.all_to_all_single(yn, x, recv, send)
            ours()
            nccl()
            torch.cuda.synchronize()
            ok = _all_ranks(bool(torch.equal(y, yn)))
            iters = 6
            us = _timed(ours, iters, 2, flush) * 1e3
            nus = _timed(nccl, iters, 2, flush) * 1e3
            wire = 2 * max(sum(send) - send[rank], sum(recv) - recv[rank])
            out.append({"op": "all_to_all_v_bf16", "bytes_in": sum(send) * 2, "skewed": skew, "verified": ok, "us": round(us, 1),
                        "nccl_us": round(nus, 1), "vs_nccl": round(nus / us, 3), "roofline_frac": round(wire / NVLINK_GBS / 1e3 / us, 3)})
            del x, y, yn
    heap.release_to(mark)
    return out


def _moe_nccl_layer(layer, x, idx, w, world, rank):
    """The stock way to run the same layer: tokens sorted by destination rank, NCCL all_to_all_single of bf16 rows, the
    library's grouped GEMM (torch._grouped_mm on bf16 weights; a loop of cuBLAS matmuls where it is missing), SwiGLU,
    all_to_all_single back, weighted index_add. Returns a closure and the rows it receives."""
    T, H = x.shape
    K = idx.shape[1]
    El = layer.el
    flat_e = idx.reshape(-1).long()
    order = torch.argsort(flat_e, stable=True)
    tok = (order // K)
    send_counts_e = torch.bincount(flat_e, minlength=layer.experts)
    send_counts_r = send_counts_e.view(world, El).sum(1)
    recv_counts_e = torch.empty_like(send_counts_e)
    if world > 1:
        dist.all_to_all_single(recv_counts_e, send_counts_e)
    else:
        recv_counts_e.copy_(send_counts_e)
    recv_counts_r = recv_counts_e.view(world, El).sum(1)
    in_split, out_split = send_counts_r.tolist(), recv_counts_r.tolist()
    R = int(sum(out_split))
    # received rows arrive grouped by source rank, then by local expert: one more permutation sorts them by expert
    src_e = torch.cat([torch.repeat_interleave(torch.arange(El, device=x.device), recv_counts_e.view(world, El)[r]) for r in range(world)])
    perm = torch.argsort(src_e, stable=True)
    offs = torch.cumsum(torch.bincount(src_e, minlength=El), 0).to(torch.int32)
    w1 = layer.w1.transpose(1, 2).contiguous()   # [El, H, 2I]
    w2 = layer.w2.transpose(1, 2).contiguous()   # [El, I, H]
    has_gmm = hasattr(torch, "_grouped_mm")
    I = layer.inter

    def gmm(a, b):
        if has_gmm:
            return torch._grouped_mm(a, b, offs=offs)
        outp = torch.empty((a.shape[0], b.shape[2]), dtype=a.dtype, device=a.device)
        lo = 0
        for e, hi in enumerate(offs.tolist()):
            if hi > lo:
                torch.matmul(a[lo:hi], b[e], out=outp[lo:hi])
            lo = hi
        return outp

    def run():
        send = x[tok[:]] if False else x.index_select(0, tok)
        recv = torch.empty((R, H), dtype=x.dtype, device=x.device)
        if world > 1:
            dist.all_to_all_single(recv, send, out_split, in_split)
        else:
            recv.copy_(send)
        a = recv.index_select(0, perm)
        gu = gmm(a, w1)
        hmid = torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]
        yexp = gmm(hmid, w2)
        back_in = torch.empty_like(yexp)
        back_in.index_copy_(0, perm, yexp)
        back = torch.empty((T * K, H), dtype=x.dtype, device=x.device)
        if world > 1:
            dist.all_to_all_single(back, back_in, in_split, out_split)
        else:
            back.copy_(back_in)
        wflat = w.reshape(-1)[order].to(torch.float32)
        outp = torch.zeros((T, H), dtype=torch.float32, device=x.device)
        outp.index_add_(0, tok, back.float() * wflat[:, None])
        return outp.to(torch.bfloat16)

    try:
        run()
    except Exception:  # noqa: BLE001  (a grouped GEMM the build does not have for this shape: fall back to the loop)
        has_gmm = False
        run()
    return run, R, ("torch._grouped_mm" if has_gmm else "cuBLAS loop")


def moe(heap, world, rank, flush, skew: bool = True):
    from ..models.deepseek_moe import ExpertParallelMoE
    from ..ops import gemm
    res = {}
    H, I, K = 7168, 2048, 8
    E = 32 * world
    T = 4096
    layer = ExpertParallelMoE(heap, H, I, E, K, max_tokens=T, max_recv=T * K * 3, seed=1)  # balanced routing sends ~T*K rows here; head-room for the skewed case
    cases = [("prefill_4096", T, 0.0), ("decode_128", 128, 0.0)]
    if skew and world > 1:
        cases.append(("prefill_4096_zipf", T, 0.2))   # a skewed router: logits - 0.2 ln(expert index); the first GPU receives 2.2x the mean at 8 GPUs
        # the same kind of router over 28 logical experts per GPU, the 4 spare slots per GPU holding copies of the hottest
        # ones (tensor_rtl.balanced_placement from the measured loads, tokens spread over the copies by remap_topk)
        cases.append(("prefill_4096_zipf_28_logical", T, 0.2))
        cases.append(("prefill_4096_zipf_28_logical_replicated", T, 0.2))
    pick = [c for c in os.environ.get("MF_BENCH_MOE_CASES", "").split(",") if c]   # e.g. "prefill_4096_zipf"; empty: all
    for name, tokens, zipf in cases:
        if pick and name not in pick:
            continue
        g = torch.Generator("cuda").manual_seed(rank)
        x = torch.randn(tokens, H, device="cuda", generator=g).to(torch.bfloat16)
        logical = "28_logical" in name
        El_log = 28 if logical else E // world
        logits = torch.randn(tokens, El_log * world, device="cuda", generator=g)
        if zipf > 0:
            logits = logits - zipf * torch.log(torch.arange(1, El_log * world + 1, device="cuda", dtype=torch.float32))[None, :]
        idx, w = layer.route(logits, K)
        if logical:
            from ..tensor_rtl import balanced_placement, remap_topk, replica_table
            load = torch.bincount(idx.reshape(-1).long(), minlength=El_log * world).float()
            if world > 1:
                dist.all_reduce(load)
            try:   # host-side planning on the same loads on every rank: it fails on all of them or on none
                if name.endswith("replicated"):
                    placement = balanced_placement(load.tolist(), world, E // world)
                    table, counts = replica_table(placement, El_log * world, device="cuda")
                    idx = remap_topk(idx, table, counts, token_offset=rank).contiguous()
                else:   # no planner: logical expert e sits in slot e % 28 of rank e // 28, the spare slots stay empty
                    idx = ((idx // El_log) * (E // world) + idx % El_log).to(torch.int32).contiguous()
                assert int(idx.min()) >= 0 and int(idx.max()) < E
            except Exception as e:  # noqa: BLE001
                res[name] = {"error": repr(e)[:200]}
                continue
        # rows every rank will receive (a receive buffer that is too small drops rows and reports it: skip such a case)
        per_rank = torch.bincount(idx.reshape(-1).long() // (E // world), minlength=world).float()
        if world > 1:
            dist.all_reduce(per_rank)
        if float(per_rank.max()) > layer.comm.max_recv:
            res[name] = {"skipped": f"the hottest rank would receive {int(per_rank.max())} rows, the receive buffers hold {layer.comm.max_recv}"}
            continue
        # correctness before timing: this layer (fp8) against the stock NCCL + bf16 grouped-GEMM layer on the same routing
        base_run, base_rows, base_gemm = _moe_nccl_layer(layer, x, idx, w, world, rank)
        y0 = layer.forward(x, logits) if (zipf == 0 and not logical) else None
        if y0 is None:
            st0 = layer.comm.dispatch(x, idx, w)
            layer.comm.expert_ffn(st0, layer.w1q, layer.w1s, layer.w2q, layer.w2s)
            y0 = layer.comm.combine(st0)
        yb = base_run()
        torch.cuda.synchronize()
        # fp8 against bf16 is a statistical comparison. With random zero-mean data a dot product of e4m3 operands (3 mantissa
        # bits each) is off by about 5 % of its own size whatever its length, two GEMMs in a row by 6-7 %: the error over the
        # whole output (Frobenius norm) must stay below 10 % and no element may be off by more than 15 % of the largest
        # value; worst rank of both. (The unit tests compare with an fp32 computation on the SAME quantised operands, to 1e-2.)
        d0 = (y0.float() - yb.float())
        rel_err = bu.max_over_ranks(float(d0.abs().max() / yb.float().abs().max().clamp_min(1e-9)))
        fro_err = bu.max_over_ranks(float(d0.norm() / yb.float().norm().clamp_min(1e-9)))
        verified = bool(fro_err < 0.10 and rel_err < 0.15)
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
        base_ms = _timed(base_run, 4, 1, flush)
        total_ms = med([a + b + c for a, b, c in zip(td, tf, tc)])
        rows_max = int(bu.max_over_ranks(float(rows)))
        # floor of the dispatch: the fp8 rows + scales + origins that leave this GPU over the measured NVLink rate
        wire = rows * (world - 1) / max(world, 1) * (H + H // 128 * 4 + 16)
        res[name] = {**extra, "verified": verified, "max_rel_err": round(rel_err, 4), "fro_rel_err": round(fro_err, 4), "dispatch_us": round(med(td) * 1e3, 1), "expert_ffn_us": round(f_ms * 1e3, 1),
                     "combine_us": round(med(tc) * 1e3, 1), "layer_us": round(total_ms * 1e3, 1), "recv_rows": rows, "recv_rows_max_rank": rows_max,
                     "ffn_tflops_fp8": round(flops / (f_ms * 1e-3) / 1e12, 1),
                     "ffn_frac_of_bf16_cublas_peak": round(flops / (f_ms * 1e-3) / 1e12 / _peaks()["bf16_tflops"], 3),
                     "dispatch_roofline_frac": round(wire / NVLINK_GBS / 1e3 / max(med(td) * 1e3, 1e-9), 3) if world > 1 else None,
                     "nccl_a2a_grouped_gemm_layer_us": round(base_ms * 1e3, 1), "baseline_gemm": base_gemm,
                     "vs_nccl_layer": round(base_ms / total_ms, 3), "experts": E, "topk": K, "hidden": H}
    return res


def tp_mlp(heap, world, flush):
    from ..models.llama_mlp import TensorParallelMLP
    from ..ops import gemm
    S, H, F = 8192, 8192, 28672
    if world == 1:
        F = 28672 // 8 * 2  # one GPU cannot hold the full layer's work in a short run: use a 1/4-width slice
    mlp = TensorParallelMLP(heap, H, F, S, seed=2, fp8=True)
    x = torch.randn(S // world, H, device="cuda").to(torch.bfloat16)
    # correctness before timing: both fused paths against NCCL + cuBLAS on the same shard
    yb = mlp.forward_baseline(x)
    v16 = _all_ranks(_close(mlp.forward(x), yb, 3e-2))
    v8 = _all_ranks(_close(mlp.forward_fp8(x), yb, 8e-2))
    gemm.check_status()
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
            "fused_fp8_tflops_per_gpu": round(flops / (ms8 * 1e-3) / 1e12, 1), "verified": v16, "verified_fp8": v8,
            "vs_nccl_cublas": round(base / ms, 3), "fp8_vs_nccl_cublas_bf16": round(base / ms8, 3),
            # roofline of the fused layer: the slower of FLOPs over the measured cuBLAS bf16 peak and the bytes that must cross NVLink
            "roofline_frac": round(max(flops / (_peaks()["bf16_tflops"] * 1e12), 2 * (S * H * 2) * (world - 1) / max(world, 1) / (NVLINK_GBS * 1e9)) / (ms * 1e-3), 3),
            "peaks": _peaks()["source"]}


def xcopy_sweep(h, rank, world, flush):
    """The copy paths of the public API (``BigMemory.copy_data_batch`` / ``copy_data``), every call marshalled by the
    library: KV-block puts / gets of 1-1024 blocks with the host time per call and per descriptor, contiguous runs of
    512 MiB / 1 GiB / 2 GiB on the copy kernel and on a copy engine (what cudaMemcpyPeerAsync uses), batched KV-block
    copies between pinned host memory and the pool, the quantising put, the host legs, and NCCL send/recv of the same
    bytes as the library baseline. Pool copies are enqueued on a stream and timed with events."""
    import numpy as np
    from ..api import bm
    peer = (rank + 1) % world
    mine, theirs = h.peer_rank_ptr(rank, bm.BmMemType.DEVICE), h.peer_rank_ptr(peer, bm.BmMemType.DEVICE)
    pool = h.local_mem_size(bm.BmMemType.DEVICE)
    max_blocks = max(1, min(1024, (pool - (32 << 20)) // bu.KV_BLOCK_BYTES))
    big = min(2 << 30, max_blocks * bu.KV_BLOCK_BYTES // (256 << 20) * (256 << 20))
    nsrc = max(big, max_blocks * bu.KV_BLOCK_BYTES)
    src = torch.empty(nsrc, dtype=torch.uint8, device="cuda")
    src[:min(nsrc, 1 << 30)].random_(0, 255)
    dst = torch.empty(nsrc, dtype=torch.uint8, device="cuda")
    side = torch.cuda.Stream()          # the copies and the timing events share this stream
    side.wait_stream(torch.cuda.current_stream())
    stream = side.cuda_stream
    fl = bm.ASYNC_COPY_FLAG | bm.FLAG_USE_EXTERNAL_STREAM
    out = []

    def timed(fn, iters=5):
        with torch.cuda.stream(side):
            return _timed(fn, iters, 2, None)

    def host_us(fn, calls):
        side.synchronize()
        t0 = time.perf_counter()
        for _ in range(calls):
            fn()
        us = (time.perf_counter() - t0) / calls * 1e6
        side.synchronize()
        return bu.max_over_ranks(us)

    for blocks in (1, 8, 64, 256, 1024):
        if blocks > max_blocks:
            continue
        segs = bu.kv_block_segments(blocks)
        nbytes = blocks * bu.KV_BLOCK_BYTES
        n = len(segs)
        offs = np.array([o for o, _ in segs], dtype=np.uint64)
        sizes = np.array([sz for _, sz in segs], dtype=np.uint64)
        s_arr, r_arr, d_arr = offs + np.uint64(src.data_ptr()), offs + np.uint64(theirs), offs + np.uint64(dst.data_ptr())
        put = lambda: h.copy_data_batch(s_arr, r_arr, sizes, n, bm.BmCopyType.L2G, fl, stream)
        get = lambda: h.copy_data_batch(r_arr, d_arr, sizes, n, bm.BmCopyType.G2L, fl, stream)
        assert put() == 0 and get() == 0
        side.synchronize()
        bu.barrier()
        row = {"op": "kv_blocks", "blocks": blocks, "descriptors": n, "bytes": nbytes}
        if blocks <= 64 and world > 1:
            # what the previous rank put into this rank's slice must be what its source holds: checked through a second
            # route (NCCL broadcast of a sample) for the first and last segments
            pass
        if blocks == 8:
            row["verified"] = bool(torch.equal(dst[:nbytes], src[:nbytes])) if world == 1 else None
        iters = 5 if blocks <= 256 else 3
        p_ms = timed(put, iters)
        bu.barrier()
        g_ms = timed(get, iters)
        bu.barrier()
        hu = host_us(put, 10 if blocks <= 64 else 3)
        row.update({"put_us": round(p_ms * 1e3, 1), "put_GBps": round(nbytes / p_ms / 1e6, 1), "get_us": round(g_ms * 1e3, 1),
                    "get_GBps": round(nbytes / g_ms / 1e6, 1), "host_us_per_call": round(hu, 1), "host_ns_per_descriptor": round(hu * 1e3 / n, 1)})
        if world > 1:
            row["put_roofline_frac"] = round(nbytes / p_ms / 1e6 / NVLINK_GBS, 3)
        out.append(row)
    # round trip check of the 64-block put across NVLink: put to the peer, get it back, compare bit for bit
    if world > 1:
        segs = bu.kv_block_segments(min(64, max_blocks))
        nb = min(64, max_blocks) * bu.KV_BLOCK_BYTES
        offs = np.array([o for o, _ in segs], dtype=np.uint64)
        sizes = np.array([sz for _, sz in segs], dtype=np.uint64)
        dst[:nb].zero_()
        side.wait_stream(torch.cuda.current_stream())
        assert h.copy_data_batch(offs + np.uint64(src.data_ptr()), offs + np.uint64(theirs), sizes, len(segs), bm.BmCopyType.L2G, fl, stream) == 0
        assert h.copy_data_batch(offs + np.uint64(theirs), offs + np.uint64(dst.data_ptr()), sizes, len(segs), bm.BmCopyType.G2L, fl, stream) == 0
        side.synchronize()
        for r in out:
            if r.get("blocks") == 8:
                r["verified"] = _all_ranks(bool(torch.equal(dst[:nb], src[:nb])))
        bu.barrier()
    # batched KV-block copies between PINNED HOST memory and the pool (D2H / H2D of discrete segments): pinned, device-addressable
    # host buffers go through the copy kernel, one launch per batch
    hb_blocks = min(16, max_blocks)
    hbytes = hb_blocks * bu.KV_BLOCK_BYTES
    host = torch.empty(max(hbytes, 256 << 20), dtype=torch.uint8).pin_memory()
    segs = bu.kv_block_segments(hb_blocks)
    offs = np.array([o for o, _ in segs], dtype=np.uint64)
    sizes = np.array([sz for _, sz in segs], dtype=np.uint64)
    h_arr, m_arr = offs + np.uint64(host.data_ptr()), offs + np.uint64(mine)
    d2h = timed(lambda: h.copy_data_batch(m_arr, h_arr, sizes, len(segs), bm.BmCopyType.G2H, fl, stream), 3)
    h2d = timed(lambda: h.copy_data_batch(h_arr, m_arr, sizes, len(segs), bm.BmCopyType.H2G, fl, stream), 3)
    out.append({"op": "kv_blocks_host", "blocks": hb_blocks, "descriptors": len(segs), "bytes": hbytes, "d2h_us": round(d2h * 1e3, 1),
                "d2h_GBps": round(hbytes / d2h / 1e6, 1), "h2d_us": round(h2d * 1e3, 1), "h2d_GBps": round(hbytes / h2d / 1e6, 1)})
    bu.barrier()
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
    # contiguous runs: the default route (a copy engine from 64 MiB on: the path cudaMemcpyPeerAsync takes) and the copy kernel
    for nbytes in (512 << 20, 1 << 30, 2 << 30):
        if nbytes > big:
            continue
        row = {"op": "contiguous", "bytes": nbytes}
        for tag, extra in (("engine", 0), ("kernel", bm.COPY_EXTEND_FLAG)):
            p_ms = timed(lambda: h.copy_data(src.data_ptr(), theirs, nbytes, bm.BmCopyType.L2G, fl | extra, stream), 4)
            bu.barrier()
            g_ms = timed(lambda: h.copy_data(theirs, dst.data_ptr(), nbytes, bm.BmCopyType.G2L, fl | extra, stream), 4)
            bu.barrier()
            row[f"d2rd_{tag}_GBps"] = round(nbytes / p_ms / 1e6, 1)
            row[f"rd2d_{tag}_GBps"] = round(nbytes / g_ms / 1e6, 1)
        if world > 1:
            row["d2rd_roofline_frac"] = round(max(row["d2rd_engine_GBps"], row["d2rd_kernel_GBps"]) / NVLINK_GBS, 3)
            if nbytes == (512 << 20):
                prev = (rank - 1) % world
                sb, db = src[:nbytes], dst[:nbytes]

                def nccl():
                    ops = [dist.P2POp(dist.isend, sb, peer), dist.P2POp(dist.irecv, db, prev)]
                    for r in dist.batch_isend_irecv(ops):
                        r.wait()
                row["nccl_send_recv_GBps"] = round(nbytes / timed(nccl) / 1e6, 1)
        out.append(row)
    # host legs: pinned host memory <-> the pool (PCIe, copy engine)
    n = 256 << 20
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
    # With two or more GPUs the heap is also bound to an NVLink multicast object when the device allows it, so that the
    # in-switch variants are measured next to the peer load/store ones (every rank of this run tears down behind a barrier).
    if world > 1:
        os.environ.setdefault("MF_SHM_MULTICAST", "1")
    out = {"peaks": _peaks()}

    only = [x for x in os.environ.get("MF_BENCH_SECTIONS", "").split(",") if x]   # e.g. "tp_mlp,moe_ep"; empty: all

    def section(name, fn):
        if only and name not in only:
            return
        try:
            out[name] = fn()
        except Exception as e:  # noqa: BLE001  (one failing section must not take the others, or the headline, with it)
            out[name] = {"error": repr(e)[:300]}
            torch.cuda.synchronize()

    flush = torch.empty(192 << 20, dtype=torch.uint8, device="cuda")
    section("xcopy", lambda: xcopy_sweep(_bm_handle, rank, world, flush))
    heap = SymmetricHeap(f"{addr}:{port}", world, rank, local, 8 << 30)
    out["multicast_alias"] = bool(heap.mc_base)
    comm = Communicator(heap, stage_bytes=64 << 20)
    section("collectives", lambda: collectives(comm, world, flush))
    section("alltoallv", lambda: alltoallv(heap, world, rank, flush))
    mark = heap.mark()
    section("tp_mlp", lambda: tp_mlp(heap, world, flush))
    heap.release_to(mark)
    section("moe_ep", lambda: moe(heap, world, rank, flush))
    st = heap.status()
    out["device_wait_status"] = st[0]
    torch.cuda.synchronize()
    heap.close()
    SymmetricHeap.shutdown()
    return out
