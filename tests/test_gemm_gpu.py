"""GPU parity of the tcgen05 bf16 GEMM against a PyTorch fp32 expression, in the style of the reference's
own GEMM test (test/examples/gemm/amdgpu/test_amdgpu_gemm.py:15-31), with a tighter tolerance."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gemm(built_lib):
    from avelang_b200 import gemm
    return gemm


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 128, 128), (256, 512, 2048), (1024, 1544, 2048),
                                   (200, 72, 136), (4096, 12352, 2048), (1, 8, 8)])
def test_gemm_matches_fp32_matmul(gemm, m, n, k):
    torch.manual_seed(0)
    A = torch.randn(m, k, device="cuda").bfloat16()
    B = (torch.randn(n, k, device="cuda") * 0.02).bfloat16()
    C = gemm.gemm_pipeline_transposed_b(A, B)
    ref = A.float() @ B.float().T
    err = (C.float() - ref.bfloat16().float()).norm() / ref.norm()
    assert torch.allclose(C.float(), ref, rtol=1e-1, atol=1e-1)  # the reference's own gate
    assert err < 2e-3, f"rel-L2 {err:.3e}"
    torch.cuda.synchronize()


def test_gemm_out_and_strided_rows(gemm):
    torch.manual_seed(1)
    A = torch.randn(384, 512, device="cuda").bfloat16()[:, :256]      # row stride 512
    B = torch.randn(320, 256, device="cuda").bfloat16()
    out = torch.zeros(384, 640, dtype=torch.bfloat16, device="cuda")[:, :320]
    gemm.gemm_pipeline_transposed_b(A, B, out=out)
    ref = A.float() @ B.float().T
    assert (out.float() - ref.bfloat16().float()).norm() / ref.norm() < 2e-3


def test_gemm_rejects_bad_arguments(gemm):
    A = torch.zeros(128, 64, device="cuda")
    with pytest.raises(ValueError, match="A must have dtype torch.bfloat16"):
        gemm.gemm_pipeline_transposed_b(A, A)
    A = A.bfloat16()
    with pytest.raises(ValueError, match="out must have shape"):
        gemm.gemm_pipeline_transposed_b(A, A, out=torch.zeros(1, 1, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(ValueError, match="multiple of 8"):
        gemm.gemm_pipeline_transposed_b(A[:, :60], A[:, :60])
