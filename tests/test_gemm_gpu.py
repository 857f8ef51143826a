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


@pytest.mark.parametrize("M,N,K,W", [(300, 264, 256, 2), (1000, 2048, 512, 4), (40, 64, 64, 4)])
def test_row_parallel_gemm_with_fused_sum_ranks_on_one_gpu(gemm, M, N, K, W):
    """Ranks emulated by as many sets of buffers on one GPU (the kernels never wait on one another, so running the
    ranks' phases one after the other is the same computation): each "rank" multiplies its K slice, its GEMM epilogue
    stores every row into the owner's staging slot, then each owner sums its rows and stores them into both results."""
    from avelang_b200 import gdn
    torch.manual_seed(5)
    # (300, 264): ragged, rows_per_owner = 150 cuts a 128-row tile and N has a narrow last tile; (40, .., 4): 10 rows per owner
    A = torch.randn(M, K, device="cuda").bfloat16()
    B = (0.1 * torch.randn(N, K, device="cuda")).bfloat16()
    rpo = (M + W - 1) // W
    stages = [torch.full((W, rpo, N), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(W)]
    outs = [torch.zeros(M, N, device="cuda", dtype=torch.bfloat16) for _ in range(W)]
    sp = torch.tensor([s.data_ptr() for s in stages], dtype=torch.int64, device="cuda")
    op = torch.tensor([o.data_ptr() for o in outs], dtype=torch.int64, device="cuda")
    ks = [slice(r * K // W, (r + 1) * K // W) for r in range(W)]
    for r in range(W):
        gemm.gemm_scatter_to_owners(A[:, ks[r]], B[:, ks[r]], stages[r], sp, r)
    for r in range(W):
        gemm.reduce_push_to_all(stages[r], op, outs[r], r)
    torch.cuda.synchronize()
    assert gdn.read_status() == 0
    parts = [gemm.gemm_pipeline_transposed_b(A[:, ks[r]].contiguous(), B[:, ks[r]].contiguous()) for r in range(W)]
    acc = torch.zeros(M, N, device="cuda")
    for part in parts:                      # bf16 partials, fp32 sum in slot order, one rounding
        acc = acc + part.float()
    want = acc.bfloat16()
    assert all(torch.equal(o, want) for o in outs)
    ref = A.float() @ B.float().T
    assert ((outs[0].float() - ref).norm() / ref.norm()).item() < 5e-3
    with pytest.raises(ValueError):
        gemm.gemm_scatter_to_owners(A, B, stages[0][:, : rpo - 1].contiguous(), sp, 0)   # the owners' rows cannot hold M
