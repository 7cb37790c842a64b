"""zbal on a GPU: the torch.distributed backend, the symmetric allocator under PyTorch, the MoE Buffer.

Each scenario runs in child processes (zbal bootstraps once per process). With one GPU the world has one
rank, which still drives every kernel; the multi-GPU test runs real ranks over NVLink and compares with
values computed locally from the ranks' seeds."""
import os

import pytest
import torch

from conftest import free_port
from mp_util import run_ranks

pytestmark = pytest.mark.gpu


def _draw(r, n, dtype=torch.float32):
    import torch
    return torch.randn(n, device="cuda", generator=torch.Generator("cuda").manual_seed(77 * r + 5)).to(dtype)


def _pg_scenario(rank, world, port, impl, sync):
    import torch
    import torch.distributed as dist
    os.environ["ZBAL_PG_IMPL"] = impl
    import memfabric_hybrid_b200.zbal as zbal
    dev = rank % torch.cuda.device_count()
    torch.cuda.set_device(dev)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    assert zbal.zbal_init(world, dev, rank, 512 << 20, ip_port=f"127.0.0.1:{port}", start_config_server=True)
    dist.init_process_group("zbal", init_method=f"tcp://127.0.0.1:{port + 1}", rank=rank, world_size=world)
    if impl == "native":   # a c10d::Backend from lib/_zbal_c10d.so under torch's own ProcessGroup
        pg = dist.group.WORLD._get_backend(torch.device("cuda"))
        assert type(pg).__module__ == "_zbal_c10d" and pg.comm_name() == "zbal_world"
    else:
        pg = dist.group.WORLD
        assert isinstance(pg, zbal.ProcessGroupZBAL)

    # all_reduce: sum, avg, max, in place, several sizes (one-shot and two-shot), async handle
    for n in (1, 1000, 70_000, 2_000_000):
        for dtype in (torch.float32, torch.bfloat16):
            x = _draw(rank, n, dtype)
            ref = sum(_draw(r, n, dtype).float() for r in range(world))
            dist.all_reduce(x)
            torch.testing.assert_close(x.float(), ref, rtol=2e-2, atol=2e-2 * world)
    x = _draw(rank, 4096)
    w = dist.all_reduce(x, op=dist.ReduceOp.MAX, async_op=True)
    w.wait()
    torch.testing.assert_close(x, torch.stack([_draw(r, 4096) for r in range(world)]).max(0).values)
    x = _draw(rank, 4096)
    dist.all_reduce(x, op=dist.ReduceOp.AVG)
    torch.testing.assert_close(x, sum(_draw(r, 4096) for r in range(world)) / world, rtol=1e-5, atol=1e-5)

    # all_gather (tensor and list forms), reduce_scatter (tensor form), broadcast, scatter, gather
    shard = _draw(rank, 3000)
    full = torch.empty(world * 3000, device="cuda")
    dist.all_gather_into_tensor(full, shard)
    assert torch.equal(full, torch.cat([_draw(r, 3000) for r in range(world)]))
    parts = [torch.empty(3000, device="cuda") for _ in range(world)]
    dist.all_gather(parts, shard)
    assert all(torch.equal(parts[r], _draw(r, 3000)) for r in range(world))
    big = _draw(rank, world * 5000)
    mine = torch.empty(5000, device="cuda")
    dist.reduce_scatter_tensor(mine, big)
    ref = sum(_draw(r, world * 5000) for r in range(world))[rank * 5000:(rank + 1) * 5000]
    torch.testing.assert_close(mine, ref, rtol=1e-5, atol=1e-5)
    b = _draw(rank, 10_000).to(torch.int64) if False else _draw(rank, 10_000)
    dist.broadcast(b, src=world - 1)
    assert torch.equal(b, _draw(world - 1, 10_000))
    got = torch.empty(777 * 2, device="cuda")
    src = [(_draw(0, 777 * 2) + r) for r in range(world)] if rank == 0 else None
    dist.scatter(got, src, src=0)
    assert torch.equal(got, _draw(0, 777 * 2) + rank)
    outs = [torch.empty(100, device="cuda") for _ in range(world)] if rank == 0 else None
    dist.gather(_draw(rank, 100), outs, dst=0)
    if rank == 0:
        assert all(torch.equal(outs[r], _draw(r, 100)) for r in range(world))

    # all_to_all_single with uneven splits: rank r sends (p + 1) rows of 8 to peer p
    rows_out = [p + 1 for p in range(world)]
    send = torch.cat([torch.full((p + 1, 8), float(rank * 100 + p), device="cuda") for p in range(world)])
    recv = torch.empty(((rank + 1) * world, 8), device="cuda")
    dist.all_to_all_single(recv, send, output_split_sizes=[rank + 1] * world, input_split_sizes=rows_out)
    exp = torch.cat([torch.full((rank + 1, 8), float(p * 100 + rank), device="cuda") for p in range(world)])
    assert torch.equal(recv, exp)

    # an int64 tensor is not reducible by the kernels: the NCCL fallback must give the right answer
    if world > 1:
        cnt = torch.full((5,), rank + 1, device="cuda", dtype=torch.int64)
        dist.all_reduce(cnt)
        assert cnt[0].item() == sum(range(1, world + 1))
        # point to point around the ring, and a strided sub-group
        msg, box = torch.full((50_000,), float(rank), device="cuda"), torch.empty(50_000, device="cuda")
        nxt, prv = (rank + 1) % world, (rank - 1) % world
        if rank % 2 == 0:
            dist.send(msg, nxt)
            dist.recv(box, prv)
        else:
            dist.recv(box, prv)
            dist.send(msg, nxt)
        assert torch.equal(box, torch.full_like(box, float(prv)))
        if world >= 4:
            groups = [dist.new_group([0, 2]), dist.new_group([1, 3])] if world == 4 else [dist.new_group(list(range(0, world, 2))),
                                                                                         dist.new_group(list(range(1, world, 2)))]
            g = groups[rank % 2]
            y = torch.full((3000,), float(rank), device="cuda")
            dist.all_reduce(y, group=g)
            members = dist.get_process_group_ranks(g)
            assert torch.equal(y, torch.full_like(y, float(sum(members))))
    dist.barrier()

    # DistributedDataParallel on top of the backend: parameter broadcast, bucketed all-reduce through Work futures
    from torch.nn.parallel import DistributedDataParallel as DDP

    def make():
        torch.manual_seed(1234)
        return torch.nn.Sequential(torch.nn.Linear(64, 128), torch.nn.ReLU(), torch.nn.Linear(128, 8)).cuda()
    ddp = DDP(make(), device_ids=[dev])
    ddp(_draw(rank, 32 * 64).view(32, 64)).square().mean().backward()
    ref_model = make()
    for r in range(world):
        (ref_model(_draw(r, 32 * 64).view(32, 64)).square().mean() / world).backward()
    for p, q in zip(ddp.module.parameters(), ref_model.parameters()):
        torch.testing.assert_close(p.grad, q.grad, rtol=1e-4, atol=1e-5)
    del ddp

    # tensors from the symmetric allocator: same offset on every rank, usable by torch, reused after free
    with zbal.switch_to_allocator():
        t = torch.arange(1 << 20, device="cuda", dtype=torch.float32)
        off = t.data_ptr() - zbal.zbal_get_symm_base_addr()
        assert zbal.in_symmetric_heap(t) and float(t.sum()) == float((1 << 20) * ((1 << 20) - 1) / 2)
        dist.all_reduce(t)
        assert float(t[5]) == 5.0 * world
    offs = [None] * world
    dist.all_gather_object(offs, off) if world > 1 else offs.__setitem__(0, off)
    assert len(set(offs)) == 1, f"allocation offsets differ across ranks: {offs}"
    used, total = zbal.get_heap_stats()
    assert 0 < used <= total and zbal.mem_get_info()[1] == total
    del t
    torch.cuda.synchronize()
    status = pg.device_status()
    del pg
    dist.destroy_process_group()
    zbal.zbal_uninit()
    return status[0]


@pytest.mark.parametrize("impl", ["native", "python"])
def test_process_group_single_gpu(impl):
    port = free_port()
    assert run_ranks(_pg_scenario, 1, (port, impl), timeout=300, with_barrier=True) == [0]


@pytest.mark.multigpu
@pytest.mark.parametrize("impl", ["native", "python"])
def test_process_group_multi_gpu(impl):
    n = min(torch.cuda.device_count(), 4)
    port = free_port()
    assert run_ranks(_pg_scenario, n, (port, impl), timeout=420, with_barrier=True) == [0] * n


def _graph_pool_scenario(rank, world, port, sync):
    """The symmetric heap as the process-wide allocator: a CUDA graph captured under it allocates from a private
    pool, replays with the captured addresses, and nobody else is handed the graph's blocks."""
    import gc
    import torch
    import memfabric_hybrid_b200.zbal as zbal
    zbal.switch_to_allocator(globally=True)          # first thing: before PyTorch initialises CUDA in this process
    torch.cuda.set_device(0)
    assert zbal.zbal_init(world, 0, rank, 1 << 30, ip_port=f"127.0.0.1:{port}", start_config_server=True)
    x = torch.ones(1 << 20, device="cuda")
    assert zbal.in_symmetric_heap(x)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        y = x * 2 + 1                                # temporaries and outputs of the capture: the private pool
        z = y.sum()
    st = zbal.heap_stats()
    assert st["poolCount"] == 1 and zbal.in_symmetric_heap(y)
    others = [torch.empty(1 << 20, device="cuda") for _ in range(16)]
    mine = {y.data_ptr(), z.data_ptr()}
    assert not any(o.data_ptr() in mine for o in others)
    x.fill_(3.0)
    g.replay()
    torch.cuda.synchronize()
    assert z.item() == 7.0 * (1 << 20)
    for o in others:
        o.fill_(-1.0)                                # must not disturb what the graph owns
    x.fill_(4.0)
    g.replay()
    torch.cuda.synchronize()
    assert z.item() == 9.0 * (1 << 20) and float(y[12345]) == 9.0
    parked = zbal.heap_stats()["poolCachedBytes"]    # the temporary of x * 2 was freed inside the capture
    torch.cuda.empty_cache()
    assert zbal.heap_stats()["poolCachedBytes"] == parked and zbal.heap_stats()["poolCount"] == 1
    del g, y, z
    gc.collect()
    torch.cuda.synchronize()
    assert zbal.heap_stats()["poolCount"] == 0
    del x, others, o
    torch.cuda.empty_cache()
    used, _ = zbal.get_heap_stats()
    zbal.zbal_uninit()
    return int(used > (1 << 20))   # nothing of the scenario is still held (library workspaces aside)


def test_cuda_graph_private_pool_under_global_allocator():
    port = free_port()
    assert run_ranks(_graph_pool_scenario, 1, (port,), timeout=300, with_barrier=True) == [0]


def _buffer_scenario(rank, world, port, sync):
    import torch
    import memfabric_hybrid_b200.zbal as zbal
    from memfabric_hybrid_b200.ops import gemm
    dev = rank % torch.cuda.device_count()
    torch.cuda.set_device(dev)
    assert zbal.zbal_init(world, dev, rank, 1 << 30, ip_port=f"127.0.0.1:{port}", start_config_server=True)
    T, H, K = 96, 1024, 4
    E = 8 * world
    g = torch.Generator("cuda").manual_seed(rank)
    x = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
    logits = torch.randn(T, E, device="cuda", generator=g)
    w, idx = torch.softmax(logits, -1).topk(K, dim=-1)
    idx[0, 1] = -1  # an unselected slot must be skipped everywhere
    expect = (x.float() * torch.where(idx >= 0, w, torch.zeros_like(w)).sum(-1, keepdim=True))

    for use_fp8 in (True, False):
        buf = zbal.Buffer(None, hidden=H, num_experts=E, num_topk=K, num_max_tokens=128, use_fp8=use_fp8)
        tpr, _, tpe, inr, _ = buf.get_dispatch_layout(idx, E)
        assert int(tpe.sum()) == int((idx >= 0).sum()) and inr.shape == (T, world)
        recv, recv_e, recv_w, counts, handle, _ = buf.dispatch(x, num_tokens_per_rank=tpr, is_token_in_rank=inr, num_tokens_per_expert=tpe,
                                                               topk_idx=idx, topk_weights=w)
        rows = sum(counts)
        assert len(counts) == E // world and recv_e.shape[0] == rows and recv_w.shape[0] == rows
        if use_fp8:
            q, s = recv
            rx = (q.float().view(rows, H // 128, 128) * s.view(rows, H // 128, 1)).view(rows, H)
        else:
            rx = recv.float()
        if world == 1:
            assert rows == int((idx >= 0).sum())
            # rows of local expert 0 are the tokens that chose expert 0, in token order
            toks = (idx == 0).any(-1).nonzero().flatten()
            assert counts[0] == toks.numel() and bool((recv_e[:counts[0]] == 0).all())
            torch.testing.assert_close(rx[:counts[0]], x[toks].float(), rtol=0.08 if use_fp8 else 0, atol=0.08 if use_fp8 else 0)
        # identity experts: the combined output is x times the sum of the selected weights
        out, _, _ = buf.combine(rx.to(torch.bfloat16), handle)
        torch.testing.assert_close(out.float(), expect, rtol=0.06, atol=0.06)

        # cached layout: a second tensor along the same routing (no layout pass), and a bias pair added by combine
        snap = (recv[0][:rows].clone(), recv[1][:rows].clone()) if use_fp8 else None   # the receive buffers are reused below
        x2 = (x.float() * 0.5).to(torch.bfloat16)
        recv2, recv_e2, _, _, handle2, _ = buf.dispatch(x2, handle=handle)
        assert torch.equal(recv_e2, recv_e)
        rx2 = (recv2[0][:rows].float().view(rows, H // 128, 128) * recv2[1][:rows].view(rows, H // 128, 1)).view(rows, H) if use_fp8 else recv2[:rows].float()
        bias = torch.full((T, H), 0.25, device="cuda", dtype=torch.bfloat16)
        out2, _, _ = buf.combine(rx2.to(torch.bfloat16), handle2, bias=(bias, bias))
        torch.testing.assert_close(out2.float(), expect * 0.5 + 0.5, rtol=0.06, atol=0.06)
        if use_fp8:
            # pre-quantised input (e4m3 rows + one power-of-two scale per 128 elements, made by the library's row quantiser):
            # the receivers get the same values as from the bf16 rows
            from memfabric_hybrid_b200.ops import moe as M
            xq = torch.empty((T, H), dtype=torch.uint8, device="cuda")
            xs = torch.empty((T, H // 128), dtype=torch.float32, device="cuda")
            nrows = torch.tensor([T], dtype=torch.int32, device="cuda")
            assert M._cu().mf_quant_rows_fp8(x.data_ptr(), H, nrows.data_ptr(), H, xq.data_ptr(), xs.data_ptr(), 64,
                                             torch.cuda.current_stream().cuda_stream) == 0
            first_q, first_s = snap
            again, _, _, _, _, _ = buf.dispatch((xq.view(torch.float8_e4m3fn), xs), topk_idx=idx, topk_weights=w)
            # same VALUES (a group whose largest value rounded down to 224 is re-quantised with half the scale and doubled bytes)
            deq = lambda q, sc: q.float().view(rows, H // 128, 128) * sc.view(rows, H // 128, 1)
            assert torch.equal(deq(again[0][:rows], again[1][:rows]), deq(first_q, first_s))

        # low-latency pair, weights travelling with the rows and weights applied at home
        (lrecv, lcount, lh, _, _) = buf.low_latency_dispatch(x, idx, 128, E, use_fp8=use_fp8, topk_weights=w)
        n = int(lh[1][-1])
        assert n == int(lcount.sum())
        if use_fp8:
            q, s = lrecv
            ly = (q[:n].float().view(n, H // 128, 128) * s[:n].view(n, H // 128, 1)).view(n, H).to(torch.bfloat16)
        else:
            ly = lrecv[:n].clone()
        lout, _, _ = buf.low_latency_combine(ly, idx, w, lh)
        torch.testing.assert_close(lout.float(), expect, rtol=0.06, atol=0.06)
        if use_fp8:
            # scales as exponent bytes (UE8M0), four per int32
            (pk, _, ph, _, _) = buf.low_latency_dispatch(x, idx, 128, E, use_fp8=True, round_scale=True, use_ue8m0=True)
            n8 = int(ph[1][-1])
            words = pk[1][:n8]
            assert words.dtype == torch.int32 and words.shape[1] == (H // 128 + 3) // 4
            expo = words.contiguous().view(torch.uint8)[:, :H // 128].to(torch.int32)
            torch.testing.assert_close(torch.exp2((expo - 127).float()), buf._moe.recv_scale()[:n8], rtol=0, atol=0)
        (lrecv, lcount, lh, _, _) = buf.low_latency_dispatch(x, idx, 128, E, use_fp8=use_fp8)
        n = int(lh[1][-1])
        if use_fp8:
            q, s = lrecv
            ly = (q[:n].float().view(n, H // 128, 128) * s[:n].view(n, H // 128, 1)).view(n, H).to(torch.bfloat16)
        else:
            ly = lrecv[:n].clone()
        lout, _, _ = buf.low_latency_combine(ly, idx, w, lh)
        torch.testing.assert_close(lout.float(), expect, rtol=0.06, atol=0.06)
        if use_fp8:
            # fused path with an activity mask: masked rows come back as zeros, the others are unchanged by the mask
            from memfabric_hybrid_b200.ops import moe as M
            El, I = E // world, 256
            gw = torch.Generator("cuda").manual_seed(99)          # the same expert weights on every rank's copy of the experts
            w1 = (torch.randn(El, 2 * I, H, device="cuda", generator=gw) * 0.03).to(torch.bfloat16)
            w2 = (torch.randn(El, H, I, device="cuda", generator=gw) * 0.03).to(torch.bfloat16)
            w1q, w1s = M.quantize_weight_fp8(w1)
            w1q = M.interleave_gate_up_fp8(w1q)
            w2q, w2s = M.quantize_weight_fp8(w2)
            full, _ = buf.fused_deep_moe(x, idx, w1q, w1s, w2q, w2s, w, E)
            full = full.clone()
            mask = torch.ones(T, dtype=torch.bool, device="cuda")
            mask[T // 2:] = False
            part, _ = buf.fused_deep_moe(x, idx, w1q, w1s, w2q, w2s, w, E, x_active_mask=mask)
            assert float(part[T // 2:].abs().max()) == 0.0 and float(full[T // 2:].abs().max()) > 0.0
            torch.testing.assert_close(part[:T // 2].float(), full[:T // 2].float(), rtol=1e-2, atol=1e-3)
            # shared expert: a dense SwiGLU FFN on every row, added to the routed result; against fp32 math on the
            # dequantised weights (activations are quantised per 1 x 128 on the way, hence the tolerance)
            Is = 256
            sw1 = (torch.randn(2 * Is, H, device="cuda", generator=gw) * 0.03).to(torch.bfloat16)
            sw2 = (torch.randn(H, Is, device="cuda", generator=gw) * 0.03).to(torch.bfloat16)
            s1q, s1s = M.quantize_weight_fp8(sw1)
            s2q, s2s = M.quantize_weight_fp8(sw2)

            def deq(q, sc):
                Nn, Kk = q.shape
                return (q.float().reshape(Nn // 128, 128, Kk // 128, 128) * sc[:, None, :, None]).reshape(Nn, Kk)

            pre = x.float() @ deq(s1q, s1s).t()
            ref_shared = (torch.nn.functional.silu(pre[:, :Is]) * pre[:, Is:]) @ deq(s2q, s2s).t()
            both, _ = buf.fused_deep_moe(x, idx, w1q, w1s, w2q, w2s, w, E, share_gmm1_weight=M.interleave_gate_up_fp8(s1q[None], 128)[0],
                                         share_gmm1_scale=s1s, share_gmm2_weight=s2q, share_gmm2_scale=s2s, share_gmm1_h_len=2 * Is)
            got_shared = both.float() - full.float()
            err = (got_shared - ref_shared).abs().max().item()
            assert err <= 0.06 * ref_shared.abs().max().item() + 2e-2, (err, ref_shared.abs().max().item())
            # smooth quant: rows times s before quantisation, weights divided by s: the product is unchanged (up to rounding)
            sm = torch.exp2(torch.randint(-1, 2, (H,), device="cuda", generator=gw).float())     # powers of two: exact in bf16 / fp8
            w1_s = (w1.float() / sm.view(1, 1, H)).to(torch.bfloat16)
            w1q_s, w1s_s = M.quantize_weight_fp8(w1_s)
            smoothed, _ = buf.fused_deep_moe(x, idx, M.interleave_gate_up_fp8(w1q_s), w1s_s, w2q, w2s, w, E, expert_smooth_scales=sm)
            err = (smoothed.float() - full.float()).abs().max().item()
            assert err <= 0.06 * full.float().abs().max().item() + 2e-2, (err, full.float().abs().max().item())
            # weights as lists of per-expert tensors
            listed, _ = buf.fused_deep_moe(x, idx, list(w1q), list(w1s), list(w2q), list(w2s), w, E, is_tensor_list=True)
            torch.testing.assert_close(listed.float(), full.float(), rtol=0, atol=0)
        torch.cuda.synchronize()
        gemm.check_status()
        buf.destroy()
    zbal.zbal_uninit()
    return 0


def test_buffer_single_gpu():
    port = free_port()
    assert run_ranks(_buffer_scenario, 1, (port,), timeout=300, with_barrier=True) == [0]


@pytest.mark.multigpu
def test_buffer_multi_gpu():
    n = min(torch.cuda.device_count(), 4)
    port = free_port()
    assert run_ranks(_buffer_scenario, n, (port,), timeout=420, with_barrier=True) == [0] * n


def _moe_capi_scenario(rank, world, port, sync):
    """The C entry points of the MoE path (zbal_moe_create, zbal_dispatch_*, zbal_combine_*, zbal_fused_deep_moe) through ctypes."""
    import ctypes as C
    import torch
    import memfabric_hybrid_b200.zbal as zbal
    from memfabric_hybrid_b200.zbal import _capi as K
    from memfabric_hybrid_b200.ops import moe as M
    from memfabric_hybrid_b200.ops.heap import tensor_at
    dev = rank % torch.cuda.device_count()
    torch.cuda.set_device(dev)
    assert zbal.zbal_init(world, dev, rank, 1 << 30, ip_port=f"127.0.0.1:{port}", start_config_server=True)
    l = K.lib()
    T, H, I, Kk = 64, 1024, 512, 2
    E = 4 * world
    El = E // world
    o = K.MoeOptionsC(T, H, E, Kk, 0, 0)
    moe = C.c_void_p()
    K.check(l.zbal_moe_create(l.zbal_comm_get_global(), C.byref(o), C.byref(moe)), "zbal_moe_create")
    bufs = K.MoeBuffersC()
    K.check(l.zbal_moe_get_buffers(moe, C.byref(bufs)), "get_buffers")
    assert bufs.localExperts == El and bufs.maxRecv == T * world * min(Kk, El)
    g = torch.Generator("cuda").manual_seed(rank)
    x = torch.randn(T, H, device="cuda", generator=g).to(torch.bfloat16)
    w, idx = torch.softmax(torch.randn(T, E, device="cuda", generator=g), -1).topk(Kk, dim=-1)
    idx, w = idx.to(torch.int32).contiguous(), (w / w.sum(-1, keepdim=True)).float().contiguous()
    i32 = dict(dtype=torch.int32, device="cuda")
    tpr, tpe, sidx = torch.empty(world, **i32), torch.empty(E, **i32), torch.zeros(T * Kk, **i32)
    inr = torch.empty(T, world, dtype=torch.uint8, device="cuda")
    rpe, row_off, put_off, src_off = torch.empty(El, **i32), torch.empty(El + 1, **i32), torch.empty(E, **i32), torch.empty(El * world, **i32)
    s = torch.cuda.current_stream().cuda_stream
    K.check(l.zbal_dispatch_normal_layout(moe, idx.data_ptr(), T, tpr.data_ptr(), tpe.data_ptr(), sidx.data_ptr(), inr.data_ptr(), s), "layout")
    K.check(l.zbal_dispatch_normal_notify(moe, tpe.data_ptr(), rpe.data_ptr(), row_off.data_ptr(), put_off.data_ptr(), src_off.data_ptr(), s), "notify")
    K.check(l.zbal_dispatch_normal(moe, x.data_ptr(), T, idx.data_ptr(), w.data_ptr(), sidx.data_ptr(), put_off.data_ptr(), s), "dispatch")
    torch.cuda.synchronize()
    assert int(tpe.sum()) == T * Kk
    rows = int(row_off[-1])
    q = tensor_at(bufs.recvTokens, (rows, H), torch.uint8).view(torch.float8_e4m3fn)
    sc = tensor_at(bufs.recvScales, (rows, H // 128), torch.float32)
    y = (q.float().view(rows, H // 128, 128) * sc.view(rows, H // 128, 1)).view(rows, H).to(torch.bfloat16)   # identity experts
    out = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
    K.check(l.zbal_combine_normal(moe, y.data_ptr(), H, row_off[El:].data_ptr(), 1, idx.data_ptr(), T, out.data_ptr(), s), "combine")
    torch.cuda.synchronize()
    torch.testing.assert_close(out.float(), x.float(), rtol=0.08, atol=0.08)     # the routing weights of a token sum to one
    # low-latency pair
    out.zero_()
    K.check(l.zbal_dispatch_low_latency(moe, x.data_ptr(), T, idx.data_ptr(), w.data_ptr(), sidx.data_ptr(), tpe.data_ptr(), rpe.data_ptr(),
                                        row_off.data_ptr(), put_off.data_ptr(), src_off.data_ptr(), s), "ll dispatch")
    torch.cuda.synchronize()
    rows = int(row_off[-1])
    q = tensor_at(bufs.recvTokens, (rows, H), torch.uint8).view(torch.float8_e4m3fn)
    sc = tensor_at(bufs.recvScales, (rows, H // 128), torch.float32)
    y = (q.float().view(rows, H // 128, 128) * sc.view(rows, H // 128, 1)).view(rows, H).to(torch.bfloat16)
    K.check(l.zbal_combine_low_latency(moe, y.data_ptr(), H, row_off[El:].data_ptr(), 1, idx.data_ptr(), None, T, out.data_ptr(), s), "ll combine")
    torch.cuda.synchronize()
    torch.testing.assert_close(out.float(), x.float(), rtol=0.08, atol=0.08)
    # fused path against an fp32 reference from the bf16 master weights of ALL experts (every rank can regenerate them)
    def weights(r):
        gg = torch.Generator("cuda").manual_seed(1000 + r)
        return ((torch.randn(El, 2 * I, H, device="cuda", generator=gg) * 0.02).to(torch.bfloat16),
                (torch.randn(El, H, I, device="cuda", generator=gg) * 0.02).to(torch.bfloat16))
    w1, w2 = weights(rank)
    w1q, w1s = M.quantize_weight_fp8(w1)
    w1q = M.interleave_gate_up_fp8(w1q)
    w2q, w2s = M.quantize_weight_fp8(w2)
    ws = torch.empty(int(l.zbal_fused_deep_moe_workspace(moe, I)), dtype=torch.uint8, device="cuda")
    K.check(l.zbal_fused_deep_moe(moe, x.data_ptr(), T, idx.data_ptr(), w.data_ptr(), w1q.data_ptr(), w1s.data_ptr(), w2q.data_ptr(), w2s.data_ptr(), I,
                                  ws.data_ptr(), out.data_ptr(), s), "fused")
    torch.cuda.synchronize()
    allw = [weights(r) for r in range(world)]
    ref = torch.zeros(T, H, device="cuda")
    for t in range(T):
        for k in range(Kk):
            e = int(idx[t, k])
            a1, a2 = allw[e // El][0][e % El].float(), allw[e // El][1][e % El].float()
            h = a1 @ x[t].float()
            ref[t] += w[t, k] * (a2 @ (torch.nn.functional.silu(h[:I]) * h[I:]))
    err = (out.float() - ref).abs().max().item() / max(ref.abs().max().item(), 1e-6)
    assert err < 0.1, f"fused MoE differs from the fp32 reference: {err}"
    # smooth-quant factors through the C entry point: with factors of 1 the result is bit-identical (the arithmetic of
    # the factors themselves is checked against fp32 math in the Buffer test)
    l.zbal_moe_set_smooth_scales.argtypes = [C.c_void_p, C.c_void_p]
    l.zbal_moe_set_smooth_scales.restype = C.c_int32
    ones = torch.ones(H, device="cuda")
    K.check(l.zbal_moe_set_smooth_scales(moe, ones.data_ptr()), "smooth scales")
    out1 = torch.empty_like(out)
    K.check(l.zbal_fused_deep_moe(moe, x.data_ptr(), T, idx.data_ptr(), w.data_ptr(), w1q.data_ptr(), w1s.data_ptr(), w2q.data_ptr(), w2s.data_ptr(), I,
                                  ws.data_ptr(), out1.data_ptr(), s), "fused with unit factors")
    torch.cuda.synchronize()
    assert torch.equal(out1, out)
    K.check(l.zbal_moe_set_smooth_scales(moe, None), "smooth scales off")
    st = C.c_int32(-1)
    K.check(l.zbal_moe_get_status(moe, C.byref(st)), "status")
    K.check(l.zbal_moe_destroy(moe), "destroy")
    zbal.zbal_uninit()
    return st.value


def test_moe_c_api_single_gpu():
    assert run_ranks(_moe_capi_scenario, 1, (free_port(),), timeout=300, with_barrier=True) == [0]


@pytest.mark.multigpu
def test_moe_c_api_multi_gpu():
    n = min(torch.cuda.device_count(), 4)
    assert run_ranks(_moe_capi_scenario, n, (free_port(),), timeout=420, with_barrier=True) == [0] * n


def _expand_scenario(rank, world, port, sync):
    """The symmetric heap grows by a segment while tensors live in it; a tensor of the NEW segment is all-reduced in direct
    mode (peers read it in place: p + (r - me) * stride must hold across segments) against an fp32 sum."""
    import os
    os.environ["ZBAL_ALLOC_CONF"] = "expandable_segments:True,max_segments:3"
    import torch
    import torch.distributed as dist
    import memfabric_hybrid_b200.zbal as zbal
    dev = rank % torch.cuda.device_count()
    torch.cuda.set_device(dev)
    assert zbal.zbal_init(world, dev, rank, 256 << 20, ip_port=f"127.0.0.1:{port}", start_config_server=True)
    dist.init_process_group("zbal", init_method=f"tcp://127.0.0.1:{port + 1}", rank=rank, world_size=world)
    first = zbal.heap_stats()
    assert first["segments"] == 1
    n = 24 << 20   # 96 MiB of fp32 per tensor: the third one cannot fit into what is left of the first 256 MiB segment
    with zbal.switch_to_allocator():   # only the three tensors come from the symmetric heap; temporaries below do not
        keep = [torch.full((n,), float(rank + 1 + i), device="cuda") for i in range(2)]
        grown = torch.empty((n,), device="cuda")     # makes the allocator add a segment, on every rank
    st = zbal.heap_stats()
    assert st["segments"] == 2 and st["segmentsAdded"] == 1 and st["heapSize"] > first["heapSize"]
    base = zbal.zbal_get_symm_base_addr()
    assert zbal.in_symmetric_heap(grown) and zbal.in_symmetric_heap(keep[0])
    grown.copy_(torch.randn(n, device="cuda", generator=torch.Generator("cuda").manual_seed(rank)))
    ref = sum(torch.randn(n, device="cuda", generator=torch.Generator("cuda").manual_seed(r)) for r in range(world))
    dist.all_reduce(grown)
    torch.testing.assert_close(grown, ref, rtol=1e-5, atol=1e-5)
    dist.all_reduce(keep[1])
    assert float(keep[1][7]) == float(sum(r + 2 for r in range(world)))
    off = grown.data_ptr() - base
    offs = [None] * world
    dist.all_gather_object(offs, off) if world > 1 else offs.__setitem__(0, off)
    assert len(set(offs)) == 1, f"offsets in the new segment differ across ranks: {offs}"
    del keep, grown
    torch.cuda.synchronize()
    dist.destroy_process_group()
    zbal.zbal_uninit()
    return 0


def test_heap_expands_single_gpu():
    port = free_port()
    assert run_ranks(_expand_scenario, 1, (port,), timeout=300, with_barrier=True) == [0]


@pytest.mark.multigpu
def test_heap_expands_multi_gpu():
    n = min(torch.cuda.device_count(), 4)
    port = free_port()
    assert run_ranks(_expand_scenario, n, (port,), timeout=420, with_barrier=True) == [0] * n
