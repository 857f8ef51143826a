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
// row-parallel form: each epilogue warp also has a [32 rows][128 columns] bf16 staging tile, so that rows leave as
// 256 contiguous bytes (stores of 16 bytes per row, as the plain epilogue issues them, make poor NVLink packets)
constexpr int EPI_STAGE_BYTES = 32 * 256;
constexpr size_t GEMM_SMEM_SCATTER = GEMM_SMEM + 4 * EPI_STAGE_BYTES;

// Row-parallel form: instead of one result matrix, every 128-row piece of this rank's partial product goes to the rank
// that owns those rows (rows_per_owner consecutive rows each), into slot `rank` of the owner's staging buffer
// [n_ranks][rows_per_owner][N] -- plain peer stores over NVLink from the GEMM's own epilogue, tile by tile, while the
// main loop of the next tile runs.  dst == nullptr: the ordinary single-matrix epilogue.
struct GemmScatter { const uint64_t* dst; int n_ranks, rank; int64_t rows_per_owner; };

struct TileCoord { int m, n; };
__device__ __forceinline__ TileCoord tile_coord(int tile, int mt, int nt) {
  const int per_group = GROUP_M * nt;
  const int g = tile / per_group, r = tile % per_group;
  const int rows = min(GROUP_M, mt - g * GROUP_M);
  return {g * GROUP_M + r % rows, r / rows};
}

__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_nt_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    __nv_bfloat16* __restrict__ C, int64_t M, int64_t N, int64_t K, int64_t ldc, uint32_t* status, int bn,
                    const GemmScatter sc) {
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
      if (sc.dst != nullptr) {
        // Row-parallel form: 128 columns at a time through this warp's staging tile (16-byte pieces, piece p of row r
        // at p ^ (r & 15): conflict-free both ways), then out two rows per instruction, 256 contiguous bytes each, to
        // the slot of the rank that owns the row.
        uint8_t* st = smem + STAGES * STAGE_BYTES + 256 + (warp - 2) * EPI_STAGE_BYTES;
        const int64_t row_first = (int64_t)tcd.m * BM + quarter * 32;
        const int owner0 = (int)min(row_first / sc.rows_per_owner, (int64_t)sc.n_ranks - 1);
        const int64_t boundary = (int64_t)(owner0 + 1) * sc.rows_per_owner;  // first row of the next owner
        const int halves = (int)((n_left + 127) / 128);
#pragma unroll 1
        for (int half = 0; half < halves; ++half) {
#pragma unroll 1
          for (int c4 = 0; c4 < 4; ++c4) {
            if (half * 128 + c4 * 32 >= n_left) break;
            uint32_t r[32];
            tc::tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + half * 128 + c4 * 32), r);
            tc::tmem_ld_wait();
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 pk;
              pk.x = pack_bf16x2(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]));
              pk.y = pack_bf16x2(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
              pk.z = pack_bf16x2(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
              pk.w = pack_bf16x2(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
              *reinterpret_cast<uint4*>(st + lane * 256 + (((c4 * 4 + v) ^ (lane & 15)) << 4)) = pk;
            }
          }
          if (half == halves - 1) {  // the accumulator is out of tensor memory: the next tile's MMAs may overwrite it
            tc::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&acc_empty[buf]);
          }
          __syncwarp();
          const int p = lane & 15;
          const int64_t col = (int64_t)half * 128 + p * 8;
#pragma unroll 4
          for (int it = 0; it < 16; ++it) {
            const int a = 2 * it + (lane >> 4);
            const int64_t grow = row_first + a;
            if (grow < M && col < n_left) {
              const uint4 pk = *reinterpret_cast<const uint4*>(st + a * 256 + ((p ^ (a & 15)) << 4));
              // a 32-row block meets at most two owners unless an owner has fewer than 32 rows
              const int owner = sc.rows_per_owner >= 32 ? (grow >= boundary ? owner0 + 1 : owner0)
                                                        : (int)min(grow / sc.rows_per_owner, (int64_t)sc.n_ranks - 1);
              __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(sc.dst[owner]) +
                                   ((int64_t)sc.rank * sc.rows_per_owner + (grow - (int64_t)owner * sc.rows_per_owner)) * ldc +
                                   (int64_t)tcd.n * bn + col;
              *reinterpret_cast<uint4*>(dst) = pk;
            }
          }
          __syncwarp();
        }
        continue;
      }
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

// Second phase of the row-parallel form, after every rank's first phase (a cross-rank barrier lies between): the owner
// sums its rows over the n_ranks slots of its staging buffer in fp32, in slot order (the same bits on every run),
// rounds once to bf16 and stores the row into every rank's result matrix.  One 16-byte piece per thread and step.
__global__ void __launch_bounds__(256) reduce_push_kernel(const __nv_bfloat16* __restrict__ stage, const uint64_t* __restrict__ out_peers,
                                                          int n_ranks, int rank, int64_t rows_per_owner, int64_t M, int64_t N, int64_t ldc) {
  const int64_t row0 = (int64_t)rank * rows_per_owner;
  const int64_t rows = max((int64_t)0, min(rows_per_owner, M - row0));
  const int64_t vec_per_row = N / 8, total = rows * vec_per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / vec_per_row, c = (i - r * vec_per_row) * 8;
    float2 acc[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
    for (int s = 0; s < n_ranks; ++s) {
      const uint4 v = *reinterpret_cast<const uint4*>(stage + ((int64_t)s * rows_per_owner + r) * N + c);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f = bf16x2_to_float2(w[e]);
        acc[e].x += f.x; acc[e].y += f.y;
      }
    }
    uint4 pk;
    pk.x = pack_bf16x2(acc[0].x, acc[0].y); pk.y = pack_bf16x2(acc[1].x, acc[1].y);
    pk.z = pack_bf16x2(acc[2].x, acc[2].y); pk.w = pack_bf16x2(acc[3].x, acc[3].y);
    for (int d = 0; d < n_ranks; ++d)
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(out_peers[d]) + (row0 + r) * ldc + c) = pk;
  }
}

}  // namespace

int launch_gemm_bf16_nt_impl(const AveGemmArgs& a, cudaStream_t stream, const GemmScatter& sc);
int launch_gemm_bf16_nt(const AveGemmArgs& a, cudaStream_t stream) { return launch_gemm_bf16_nt_impl(a, stream, GemmScatter{nullptr, 1, 0, 0}); }

int launch_gemm_bf16_nt_scatter(const AveGemmReduceArgs& r, cudaStream_t stream) {
  AveGemmArgs a{};
  a.struct_size = sizeof(AveGemmArgs);
  a.a = r.a; a.b = r.b; a.c = r.stage;  // the tensor-map-free C pointer is replaced per row by the owner's slot
  a.M = r.M; a.N = r.N; a.K = r.K; a.lda = r.lda; a.ldb = r.ldb; a.ldc = r.N;
  a.status = r.status;
  return launch_gemm_bf16_nt_impl(a, stream, GemmScatter{reinterpret_cast<const uint64_t*>(r.stage_peers), r.n_ranks, r.rank, r.rows_per_owner});
}

int launch_gemm_reduce_push(const AveGemmReduceArgs& r, cudaStream_t stream) {
  int dev = 0, sms = 148;
  AVE_CUDA_TRY(cudaGetDevice(&dev));
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  reduce_push_kernel<<<sms * 8, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(r.stage), reinterpret_cast<const uint64_t*>(r.out_peers),
                                                 r.n_ranks, r.rank, r.rows_per_owner, r.M, r.N, r.ldc);
  AVE_CUDA_TRY(cudaGetLastError());
  return AVE_GDN_OK;
}

int launch_gemm_bf16_nt_impl(const AveGemmArgs& a, cudaStream_t stream, const GemmScatter& sc) {
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
    AVE_CUDA_TRY(cudaFuncSetAttribute(gemm_bf16_nt_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GEMM_SMEM_SCATTER));
    attr_set_dev[dev & 63] = true;
  }
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t tiles = ((a.M + BM - 1) / BM) * ((a.N + bn - 1) / bn);
  const unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
  gemm_bf16_nt_kernel<<<grid, GEMM_THREADS, sc.dst != nullptr ? GEMM_SMEM_SCATTER : GEMM_SMEM, stream>>>(tmA, tmB, reinterpret_cast<__nv_bfloat16*>(a.c), a.M, a.N, a.K,
                                                               a.ldc, a.status, bn, sc);
  AVE_CUDA_TRY(cudaGetLastError());
  return AVE_GDN_OK;
}

}  // namespace ave
