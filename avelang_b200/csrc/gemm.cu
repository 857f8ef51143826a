// C[M,N] = A[M,K] * B[N,K]^T, bf16 operands, fp32 accumulation in tensor memory, bf16 result.
//
// Persistent kernel, one CTA per SM, 128x256 output tiles, K in steps of 64 (one 128-byte swizzle span):
//   warp 0      TMA producer: A and B tiles into a 4-stage shared-memory ring
//   warp 1      issues tcgen05.mma (128x256x16 per instruction) into one of two 256-column TMEM accumulators
//   warps 2..5  epilogue: TMEM -> registers -> bf16 -> global, overlapped with the next tile's main loop
// Tiles are walked in groups of 16 row-tiles so the A rows of a group stay in L2 while B is swept.
#include "common.cuh"
#include "tc.cuh"

namespace ave {
namespace {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int GEMM_THREADS = 192;
constexpr int GROUP_M = 16;
constexpr size_t GEMM_SMEM = (size_t)STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;

struct TileCoord { int m, n; };
__device__ __forceinline__ TileCoord tile_coord(int tile, int mt, int nt) {
  const int per_group = GROUP_M * nt;
  const int g = tile / per_group, r = tile % per_group;
  const int rows = min(GROUP_M, mt - g * GROUP_M);
  return {g * GROUP_M + r % rows, r / rows};
}

__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_nt_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    __nv_bfloat16* __restrict__ C, int64_t M, int64_t N, int64_t K, int64_t ldc, uint32_t* status, int bn) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* full = bars;                 // [STAGES]
  uint64_t* empty = bars + STAGES;       // [STAGES]
  uint64_t* acc_full = bars + 2 * STAGES;      // [2]
  uint64_t* acc_empty = bars + 2 * STAGES + 2; // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // bn: width of a column tile, a multiple of 16 up to BN chosen by the launcher so that the column tiles are of
  // (nearly) equal width; shared memory and tensor memory are laid out for BN
  const int mt = (int)((M + BM - 1) / BM), nt = (int)((N + bn - 1) / bn), kb_count = (int)((K + BK - 1) / BK);
  const int n_tiles = mt * nt;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { tc::mbar_init(&full[s], 1); tc::mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { tc::mbar_init(&acc_full[b], 1); tc::mbar_init(&acc_empty[b], 4); }
    *abort_flag = 0;
    tc::fence_barrier_init();
    tc::prefetch_tmap(&tmA);
    tc::prefetch_tmap(&tmB);
  }
  if (warp == 1) tc::tmem_alloc(tmem_slot, 512);
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int s = 0; uint32_t ph = 0;
      for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const TileCoord tcd = tile_coord(tile, mt, nt);
        for (int kb = 0; kb < kb_count; ++kb) {
          if (!tc::mbar_wait(&empty[s], ph ^ 1u, abort_flag)) goto producer_done;
          tc::mbar_expect_tx(&full[s], (uint32_t)(A_BYTES + bn * BK * 2));
          tc::tma_load_2d(smem + s * STAGE_BYTES, &tmA, &full[s], kb * BK, tcd.m * BM);
          tc::tma_load_2d(smem + s * STAGE_BYTES + A_BYTES, &tmB, &full[s], kb * BK, tcd.n * bn);
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
      }
    }
  producer_done:;
  } else if (warp == 1) {
    if (lane == 0) {
      int s = 0; uint32_t ph = 0; int local = 0;
      for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++local) {
        const uint32_t idesc = tc::idesc_f16(BM, bn, 1, 1, false, false);
        const int buf = local & 1;
        const uint32_t acc_ph = (uint32_t)(local >> 1) & 1u;
        if (!tc::mbar_wait(&acc_empty[buf], acc_ph ^ 1u, abort_flag)) break;
        tc::tc_fence_after_sync();
        const uint32_t d = tmem_base + (uint32_t)buf * BN;
        bool ok = true;
        for (int kb = 0; kb < kb_count; ++kb) {
          if (!tc::mbar_wait(&full[s], ph, abort_flag)) { ok = false; break; }
          tc::tc_fence_after_sync();
          const uint32_t a_addr = tc::smem_u32(smem + s * STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            tc::mma_ss(d, tc::smem_desc_sw128(a_addr + k * 32, 16, 1024), tc::smem_desc_sw128(b_addr + k * 32, 16, 1024), idesc,
                       (kb | k) != 0 ? 1u : 0u);
          }
          tc::mma_commit(&empty[s]);
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
        if (!ok) break;
        tc::mma_commit(&acc_full[buf]);
      }
    }
  } else {
    const int quarter = warp & 3;  // TMEM lanes this warp may touch
    int local = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++local) {
      const TileCoord tcd = tile_coord(tile, mt, nt);
      const int buf = local & 1;
      const uint32_t acc_ph = (uint32_t)(local >> 1) & 1u;
      if (!tc::mbar_wait(&acc_full[buf], acc_ph, abort_flag)) break;
      tc::tc_fence_after_sync();
      const int64_t row = (int64_t)tcd.m * BM + quarter * 32 + lane;
      __nv_bfloat16* crow = C + row * ldc + (int64_t)tcd.n * bn;
      const int64_t n_left = min((int64_t)bn, N - (int64_t)tcd.n * bn);
      const int col_groups = (int)((n_left + 31) / 32);  // 32-column groups that hold results
#pragma unroll 1
      for (int c = 0; c < col_groups; ++c) {
        uint32_t r[32];
        tc::tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + c * 32), r);
        tc::tmem_ld_wait();
        if (row < M) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const int col = c * 32 + v * 8;
            if (col + 8 <= n_left) {
              uint4 pk;
              pk.x = pack_bf16x2(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]));
              pk.y = pack_bf16x2(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
              pk.z = pack_bf16x2(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
              pk.w = pack_bf16x2(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
              *reinterpret_cast<uint4*>(crow + col) = pk;
            } else {
              for (int e = 0; e < 8; ++e)
                if (col + e < n_left) crow[col + e] = __float2bfloat16(__uint_as_float(r[v * 8 + e]));
            }
          }
        }
      }
      tc::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(&acc_empty[buf]);
    }
  }

  tc::tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag != 0 && status != nullptr) atomicOr(status, AVE_GDN_DEV_WAIT_EXPIRED);
  if (warp == 1) {
    tc::tc_fence_after_sync();
    tc::tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace

int launch_gemm_bf16_nt(const AveGemmArgs& a, cudaStream_t stream) {
  CUtensorMap tmA, tmB;
  const uint64_t dimsA[2] = {(uint64_t)a.K, (uint64_t)a.M}, strA[2] = {2, (uint64_t)a.lda * 2};
  const uint64_t dimsB[2] = {(uint64_t)a.K, (uint64_t)a.N}, strB[2] = {2, (uint64_t)a.ldb * 2};
  // Column tiles of equal width: as few tiles as BN = 256 allows, each as narrow as that count permits (a multiple of
  // 16, the granularity of the MMA's N).  N = 1544 becomes 7 tiles of 224 columns instead of 6 of 256 and one of 8,
  // whose MMAs and A-tile loads would be spent on 8 columns of output.
  const int64_t n_tiles_n = (a.N + BN - 1) / BN;
  const int bn = (int)(((a.N + n_tiles_n - 1) / n_tiles_n + 15) / 16 * 16);
  const uint32_t boxA[2] = {BK, BM}, boxB[2] = {BK, (uint32_t)bn};
  int rc = make_tmap(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(a.a), 2, dimsA, strA, boxA, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != AVE_GDN_OK) return rc;
  rc = make_tmap(&tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(a.b), 2, dimsB, strB, boxB, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != AVE_GDN_OK) return rc;
  static bool attr_set_dev[64] = {};
  int dev = 0;
  AVE_CUDA_TRY(cudaGetDevice(&dev));
  if (!attr_set_dev[dev & 63]) {
    AVE_CUDA_TRY(cudaFuncSetAttribute(gemm_bf16_nt_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GEMM_SMEM));
    attr_set_dev[dev & 63] = true;
  }
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t tiles = ((a.M + BM - 1) / BM) * ((a.N + bn - 1) / bn);
  const unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
  gemm_bf16_nt_kernel<<<grid, GEMM_THREADS, GEMM_SMEM, stream>>>(tmA, tmB, reinterpret_cast<__nv_bfloat16*>(a.c), a.M, a.N, a.K,
                                                               a.ldc, a.status, bn);
  AVE_CUDA_TRY(cudaGetLastError());
  return AVE_GDN_OK;
}

}  // namespace ave
