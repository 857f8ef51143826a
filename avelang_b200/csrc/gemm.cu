// C[M,N] = A[M,K] B[N,K]^T (bf16, fp32 accumulate).  Placeholder until the tcgen05 kernel lands.
#include "common.cuh"
namespace ave {
int launch_gemm_bf16_nt(const AveGemmArgs&, cudaStream_t) { return AVE_GDN_UNSUPPORTED; }
}  // namespace ave
