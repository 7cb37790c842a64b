"""Fused tensor-parallel MLP (all-gather->GEMM+SwiGLU, GEMM->reduce-scatter) against an fp32 reference."""
import pytest
import torch

from conftest import free_port
from mp_util import run_ranks

pytestmark = pytest.mark.gpu


def _ranks(rank, world, url, T, H, F, fused1, sync):
    import torch
    from memfabric_hybrid_b200.ops import gemm
    from memfabric_hybrid_b200.ops.heap import SymmetricHeap
    from memfabric_hybrid_b200.models.llama_mlp import TensorParallelMLP
    dev = rank % torch.cuda.device_count()
    need = (1 << 20) + 2 * T * H * 2 + 2 * T * H * 2 + (8 << 20)
    heap = SymmetricHeap(url, world, rank, dev, need)
    mlp = TensorParallelMLP(heap, H, F, T, seed=3)
    mlp.tp.plain_at_world1 = not fused1
    rows = T // world
    worst = 0.0
    for it in range(3):  # several calls: exercises the double buffering and the monotonic counters
        xs = [torch.randn(rows, H, device="cuda", generator=torch.Generator("cuda").manual_seed(50 * it + r)).to(torch.bfloat16)
              for r in range(world)]
        y = mlp.forward(xs[rank])
        torch.cuda.synchronize()
        gemm.check_status()
        # fp32 reference with every rank's weights regenerated locally
        x = torch.cat(xs).float()
        ref = torch.zeros(T, H, device="cuda")
        for r in range(world):
            g = torch.Generator("cuda").manual_seed(3 * 1000 + r)
            wg = (torch.randn(F // world, H, device="cuda", generator=g) * 0.02).to(torch.bfloat16).float()
            wu = (torch.randn(F // world, H, device="cuda", generator=g) * 0.02).to(torch.bfloat16).float()
            wd = (torch.randn(H, F // world, device="cuda", generator=g) * 0.02).to(torch.bfloat16).float()
            h = (torch.nn.functional.silu(x @ wg.t()) * (x @ wu.t())).to(torch.bfloat16).float()
            ref += h @ wd.t()
        mine = ref[rank * rows:(rank + 1) * rows]
        err = (y.float() - mine).abs().max().item()
        worst = max(worst, err / (mine.abs().max().item() + 1e-6))
    st = heap.status()[0]
    heap.close()
    SymmetricHeap.shutdown()
    return worst, st


@pytest.mark.parametrize("fused1,T", [(True, 512), (True, 384), (False, 512)], ids=["fused_cta_pairs", "fused_single_ctas", "plain_gemm"])
def test_tp_mlp_world1(fused1, T):
    """512 rows: whole 256-row tiles, the fused kernels run on CTA pairs; 384 rows: they fall back to one CTA per tile."""
    url = f"127.0.0.1:{free_port()}"
    (worst, st), = run_ranks(_ranks, 1, (url, T, 512, 1024, fused1), timeout=300, with_barrier=True)
    assert st == 0 and worst < 3e-2, (worst, st)


@pytest.mark.multigpu
def test_tp_mlp_multi_gpu():
    n = 2 if torch.cuda.device_count() < 4 else 4
    url = f"127.0.0.1:{free_port()}"
    res = run_ranks(_ranks, n, (url, 1024, 512, 2048, True), timeout=300, with_barrier=True)
    for worst, st in res:
        assert st == 0 and worst < 3e-2, res
    # shards of 384 rows are not whole 256-row tiles: the one-CTA tiling of the fused kernels
    url = f"127.0.0.1:{free_port()}"
    res = run_ranks(_ranks, n, (url, 384 * n, 512, 2048, True), timeout=300, with_barrier=True)
    for worst, st in res:
        assert st == 0 and worst < 3e-2, res


def _ranks_fp8(rank, world, url, T, H, F, sync):
    """fp8 path against an fp32 reference of the SAME quantised computation: x quantised per 1 x 128 (power-of-two scales),
    e4m3 weights with 128 x 128 scales, SwiGLU rounded to bf16 and re-quantised, partial products rounded to bf16."""
    import torch
    from memfabric_hybrid_b200.ops import gemm, moe as M
    from memfabric_hybrid_b200.ops.heap import SymmetricHeap
    from memfabric_hybrid_b200.models.llama_mlp import TensorParallelMLP
    dev = rank % torch.cuda.device_count()
    need = (1 << 20) + 2 * T * H * 2 + 2 * T * H * 2 + 2 * T * (H // 128) * 4 + (8 << 20)
    heap = SymmetricHeap(url, world, rank, dev, need)
    mlp = TensorParallelMLP(heap, H, F, T, seed=3, fp8=True)
    rows = T // world
    s = torch.cuda.current_stream().cuda_stream

    def quant(t):   # the library's row quantiser (checked on its own in test_gpu_moe)
        t = t.to(torch.bfloat16).contiguous()
        q = torch.empty(t.shape, dtype=torch.uint8, device="cuda")
        sc = torch.empty((t.shape[0], t.shape[1] // 128), dtype=torch.float32, device="cuda")
        n = torch.tensor([t.shape[0]], dtype=torch.int32, device="cuda")
        assert M._cu().mf_quant_rows_fp8(t.data_ptr(), t.shape[1], n.data_ptr(), t.shape[1], q.data_ptr(), sc.data_ptr(), 64, s) == 0
        return (q.view(torch.float8_e4m3fn).float().view(t.shape[0], -1, 128) * sc[:, :, None]).view(t.shape)

    def deq_w(q, sc):
        Nn, K = q.shape
        return (q.float().reshape(Nn // 128, 128, K // 128, 128) * sc[:, None, :, None]).reshape(Nn, K)

    worst = 0.0
    for it in range(3):
        xs = [torch.randn(rows, H, device="cuda", generator=torch.Generator("cuda").manual_seed(50 * it + r)).to(torch.bfloat16)
              for r in range(world)]
        y = mlp.forward_fp8(xs[rank])
        torch.cuda.synchronize()
        gemm.check_status()
        x = quant(torch.cat(xs))
        ref = torch.zeros(T, H, device="cuda")
        for r in range(world):
            g = torch.Generator("cuda").manual_seed(3 * 1000 + r)
            wg = (torch.randn(F // world, H, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
            wu = (torch.randn(F // world, H, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
            wd = (torch.randn(H, F // world, device="cuda", generator=g) * 0.02).to(torch.bfloat16)
            gu = deq_w(*M.quantize_weight_fp8(torch.cat([wg, wu])))
            wdd = deq_w(*M.quantize_weight_fp8(wd))
            pre = x @ gu.t()
            h = quant(torch.nn.functional.silu(pre[:, :F // world]) * pre[:, F // world:])
            ref += (h @ wdd.t()).to(torch.bfloat16).float()
        mine = ref[rank * rows:(rank + 1) * rows]
        err = (y.float() - mine).abs().max().item()
        worst = max(worst, err / (mine.abs().max().item() + 1e-6))
    st = heap.status()[0]
    heap.close()
    SymmetricHeap.shutdown()
    return worst, st


def test_tp_mlp_fp8_world1():
    url = f"127.0.0.1:{free_port()}"
    (worst, st), = run_ranks(_ranks_fp8, 1, (url, 512, 512, 1024), timeout=300, with_barrier=True)
    assert st == 0 and worst < 3e-2, (worst, st)


@pytest.mark.multigpu
def test_tp_mlp_fp8_multi_gpu():
    n = 2 if torch.cuda.device_count() < 4 else 4
    url = f"127.0.0.1:{free_port()}"
    res = run_ranks(_ranks_fp8, n, (url, 1024, 1024, 2048), timeout=300, with_barrier=True)
    for worst, st in res:
        assert st == 0 and worst < 3e-2, res
