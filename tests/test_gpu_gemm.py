"""tcgen05/TMEM GEMM kernels against fp32 PyTorch references."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 256), (256, 512, 512), (200, 320, 1024), (1024, 1024, 4096),
                                   (8, 264, 72), (4096, 7168, 2048)])
def test_gemm_bf16(M, N, K):
    from memfabric_hybrid_b200.ops import gemm
    torch.manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    b = (torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16)
    c = gemm.gemm_bf16(a, b)
    torch.cuda.synchronize()
    gemm.check_status()
    ref = a.float() @ b.float().t()
    err = (c.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 1e-2 * scale + 1e-2, f"max abs err {err} vs scale {scale}"
