"""tcgen05/TMEM GEMM kernels against fp32 PyTorch references."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 256), (256, 512, 512), (200, 320, 1024), (1024, 1024, 4096),
                                   (8, 264, 72), (4096, 7168, 2048)])
@pytest.mark.parametrize("pair", [False, True], ids=["one_cta", "cta_pair"])
def test_gemm_bf16(M, N, K, pair):
    from memfabric_hybrid_b200.ops import gemm
    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    b = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    c = gemm.gemm_bf16(a, b, pair=pair)
    torch.cuda.synchronize()
    gemm.check_status()
    ref = a.float() @ b.float().t()
    err = (c.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 1e-2 * scale + 1e-2, f"max abs err {err} vs scale {scale}"


@pytest.mark.parametrize("pair", [False, True], ids=["one_cta", "cta_pair"])
@pytest.mark.parametrize("M,F,K", [(256, 256, 512), (1000, 1024, 2048)])
def test_gemm_bf16_swiglu_epilogue(M, F, K, pair):
    """gate / up weights interleaved per 128 rows; the epilogue writes silu(gate) * up."""
    from memfabric_hybrid_b200.ops import gemm
    torch.manual_seed(M + F + K)
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    wg = (torch.randn(F, K, device="cuda") * 0.05).to(torch.bfloat16)
    wu = (torch.randn(F, K, device="cuda") * 0.05).to(torch.bfloat16)
    c = gemm.gemm_bf16(a, gemm.interleave_gate_up(wg, wu), swiglu=True, pair=pair)
    torch.cuda.synchronize()
    gemm.check_status()
    assert c.shape == (M, F)
    ref = torch.nn.functional.silu(a.float() @ wg.float().t()) * (a.float() @ wu.float().t())
    err = (c.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 1e-2 * scale + 1e-2, f"max abs err {err} vs scale {scale}"
