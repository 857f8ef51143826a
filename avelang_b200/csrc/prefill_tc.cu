// Chunked gated-delta-rule prefill on the tensor cores (d_k = d_v = 128, chunk 64).
//
// Pass 1, chunk_prep (one CTA per (chunk, value head), fully parallel, four CTAs per SM): in-chunk cumulative gate b,
//   [K; Q] K^T on tcgen05 -> A = strict_lower(beta_i e^{b_i-b_j} k_i.k_j) and P = scale * lower_incl(e^{b_i-b_j} q_i.k_j);
//   T = (I+A)^-1 by 16x16 blocks (warp-level tf32 MMAs); W^T = K^T (T diag(beta e^b))^T on tcgen05.  W^T, P and
//   Tu = T diag(beta) leave as bf16 hi+lo pairs (the tensor cores then see 16 significant bits), each as the swizzled
//   shared-memory image of its tile so that a bulk copy moves it out here and in again in pass 2, plus per-token
//   scale vectors.
// Pass 2, chunk_scan (one CTA per (sequence, value head)): the recurrence over chunks with the state kept
//   on chip, transposed (H = M^T, rows = d_v = TMEM lanes) so that every MMA has M = 128:
//     Vn^T = V^T Tu^T - H W^T             (A = V tile MN-major / H hi/lo from TMEM, B = Tu hi/lo, W^T hi/lo MN-major)
//     O^T  = qs-scaled H Q^T + Vn^T P^T   (A = H or Vn hi/lo from TMEM, B = Q or P hi/lo, K-major)
//     H   <- e^{b_C} H + Vd^T K           (A = Vd hi/lo from TMEM, B = K, MN-major), Vd_j = e^{b_C-b_j} Vn_j
//   The fp32 master copy of H lives in the chain-epilogue threads' registers; its bf16 hi/lo image is rewritten to
//   TMEM every chunk.  Four warpgroups with redistributed register budgets: control (warp 0 = TMA loader, warp 1 issues
//   the MMAs the recurrence waits for, warp 2 the output MMAs), two chain-epilogue groups (each covers all 128 TMEM
//   lanes and half of the columns), one output group.
//   With a gate tensor z the un-normalised output goes to fp32 scratch and a gated-RMSNorm launch finishes it
//   (optionally storing each row into every GPU's buffer: the fused all-gather).
// All waits are bounded; on give-up the CTA drains, frees its tensor memory and sets a status bit.
#include <mutex>

#include "common.cuh"
#include "tc.cuh"

namespace ave {
namespace {

constexpr int C = 64;     // chunk
constexpr int D = 128;    // d_k = d_v
constexpr int REC_W = C * D * 2;       // one bf16 [64][128] tile
constexpr int REC_P = C * C * 2;       // one bf16 [64][64] tile
constexpr int SCAL_FLOATS = 3 * C;     // qs[64] ks[64] decay(+pad)

struct PrepOut {
  __nv_bfloat16 *w_hi, *w_lo, *p_hi, *p_lo, *tu_hi, *tu_lo;
  float *scal;
};

struct ChunkRef { int n, b, t0, len, cis; bool ok; };  // cis: index of the chunk inside its sequence

__device__ __forceinline__ ChunkRef find_chunk(const AveGdnArgs& a, const int32_t* chunk_start, int c) {
  ChunkRef r; r.ok = false;
  if (a.cu_seqlens == nullptr) {
    const int per = (a.T + C - 1) / C;
    r.n = c / per; r.b = r.n;
    if (r.n >= a.B) return r;
    r.cis = c - r.n * per;
    r.t0 = r.cis * C; r.len = min(C, a.T - r.t0); r.ok = true;
    return r;
  }
  if (c >= chunk_start[a.n_seqs]) return r;
  const int lo = chunk_start[a.n_seqs + 1 + c];  // chunk -> sequence map, stored behind the prefix table
  const int s0 = a.cu_seqlens[lo], s1 = a.cu_seqlens[lo + 1];
  if (s0 < 0 || s1 < s0 || s1 > a.T) return r;
  r.n = lo; r.b = 0; r.cis = c - chunk_start[lo]; r.t0 = s0 + r.cis * C; r.len = min(C, s1 - r.t0); r.ok = r.len > 0;
  return r;
}

// One CTA of 1024 threads builds the chunk tables of a packed batch: chunk_start[n] = chunks of sequences 0..n-1,
// chunk_start[n_seqs] = their total, then the chunk -> sequence map and the scan's launch order.  The scratch behind the
// tables is sized for T/64 + n_seqs chunks, which holds exactly when the offsets are monotone and stay inside [0, T];
// a table that breaks this would send later sequences' records past their regions, so the whole batch is skipped
// instead: the total is stored as -1 (every CTA of the following launches tests it and leaves) and the status word gets
// AVE_GDN_DEV_BAD_SEQLEN.
__global__ void chunk_table_tc_kernel(const int32_t* __restrict__ cu_seqlens, int n_seqs, int T, int32_t* __restrict__ chunk_start,
                                      int max_chunks, uint32_t* __restrict__ status) {
  __shared__ int part[1024];
  const int per = (n_seqs + 1023) / 1024;
  const int lo = threadIdx.x * per, hi = min(lo + per, n_seqs);
  int s = 0, bad = 0;
  for (int n = lo; n < hi; ++n) {
    const int a0 = cu_seqlens[n], a1 = cu_seqlens[n + 1];
    bad |= (a0 < 0 || a1 < a0 || a1 > T) ? 1 : 0;
    s += max(0, (a1 - a0 + C - 1) / C);
  }
  part[threadIdx.x] = s;
  bad = __syncthreads_or(bad);
  if (threadIdx.x == 0) {
    int run = 0;
    for (int i = 0; i < 1024; ++i) { const int x = part[i]; part[i] = run; run += x; }
    bad |= run > max_chunks ? 1 : 0;
    chunk_start[n_seqs] = bad ? -1 : run;
    if (bad && status != nullptr) atomicOr(status, AVE_GDN_DEV_BAD_SEQLEN);
  }
  __syncthreads();
  if (bad) return;
  int run = part[threadIdx.x];
  int32_t* chunk_seq = chunk_start + n_seqs + 1;  // chunk_seq[c] = sequence that owns chunk c
  for (int n = lo; n < hi; ++n) {
    chunk_start[n] = run;
    const int cnt = max(0, (cu_seqlens[n + 1] - cu_seqlens[n] + C - 1) / C);
    for (int i = 0; i < cnt && run + i < max_chunks; ++i) chunk_seq[run + i] = n;
    run += cnt;
  }
  // Launch order of the scan's CTAs: longest sequences first, so that the last CTAs to start are short ones and the
  // SMs finish together (one CTA walks one sequence's chain).  Exact ranking up to 1024 sequences; beyond that the
  // tail is short against the total anyway and the order is the input order.
  int32_t* order = chunk_seq + max_chunks;
  __syncthreads();
  if (n_seqs <= 1024) {
    const int me = threadIdx.x;
    const int mine = me < n_seqs ? max(0, (cu_seqlens[me + 1] - cu_seqlens[me] + C - 1) / C) : -1;
    part[me] = mine;
    __syncthreads();
    if (me < n_seqs) {
      int rank = 0;
      for (int m = 0; m < n_seqs; ++m) rank += (part[m] > mine || (part[m] == mine && m < me)) ? 1 : 0;
      order[rank] = me;
    }
  } else {
    for (int n = lo; n < hi; ++n) order[n] = n;
  }
}


struct GdnMaps {
  CUtensorMap q, k, v;
};

// How one launch cuts the chunks of every sequence.
//   parts : a sequence's chunks are cut into up to `parts` consecutive parts, [part_begin[p], part_begin[p+1]), that are
//           scanned at the same time by different CTAs.  Part 0 starts from the true initial state.  A later part p runs
//           two chains: a local one from a zero state (its outputs miss the contribution of the state M0(p) that enters
//           the part) and a transition chain, the same recurrence with v = 0 started from the identity, whose state is
//           the part's transition matrix F (M_end = F M0 + local end state) and whose "output" is qt_t = scale F_t^T q_t,
//           so that the missing contribution is M0(p)^T qt_t: one GEMM per part once M0(p) is known.
//   ranges: independently, a launch covers only the chunk offsets [r0, r0 + rn) inside every part, so that pass 1 of a
//           later range runs while pass 2 walks an earlier one; a chain's state crosses launches in the carry buffer.
constexpr int MAX_PARTS = 8;
struct ScanPlan {
  int parts;
  int part_begin[MAX_PARTS + 1];  // part_begin[parts] = 1 << 24
  int r0, rn;
};
constexpr int PACK_BYTES = 2 * 128 * 128 * 2;  // bf16 hi image | lo image of one [128][128] operand
constexpr int QT_BYTES = 2 * 128 * 64 * 2;     // bf16 hi image | lo image of one chunk's qt^T [128 d_k][64 tokens]
// byte offset of the 16-byte piece (8 consecutive k) of row `row` in a K-major [128 rows][128 k] bf16 operand stored as
// two 64-wide K halves of 128-byte rows with the 128-byte swizzle (the layout tcgen05.mma reads)
__device__ __forceinline__ uint32_t kmajor_piece_off(int row, int k8) {
  return (uint32_t)((k8 >> 3) * 16384 + row * 128 + (((k8 & 7) ^ (row & 7)) << 4));
}

// ------------------------------------------------------------------------------------------------ pass 1
// Shared memory of chunk_prep (offsets from a 1024-byte aligned base).  The K and Q tiles are interleaved by
// 64-wide halves, [K_h0 | Q_h0 | K_h1 | Q_h1], so that one M = 128 MMA reads [K; Q] as its A operand (rows 0..63 =
// K, 64..127 = Q) and the K rows alone as its N = 64 B operand: lanes 0..63 of the accumulator are K K^T, lanes
// 64..127 are Q K^T.

// ---- 16x16 fp32 block algebra on legacy warp MMAs (m16n8k8 tf32), used for the triangular inverse -----------------
// Blocks live in shared memory as [16][BLK_LD] fp32.  Each product is issued as three tf32 MMAs per fragment
// (hi*hi + lo*hi + hi*lo) so the result carries fp32-level accuracy.
constexpr int BLK_LD = 20;                 // row stride (floats): conflict-free left-operand fragment loads
constexpr int BLK_FLOATS = 16 * BLK_LD;    // 320
__host__ __device__ constexpr int tri(int r, int c) { return r * (r + 1) / 2 + c; }  // lower-triangular block index

__device__ __forceinline__ uint32_t to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ void mma_tf32(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
// acc[nt] (+)= L * R for one 16x16 block pair; `lget(row, col)` returns element (row, col) of the left operand.
template <class LGet>
__device__ __forceinline__ void block_mma(float (&acc)[2][4], LGet lget, const float* __restrict__ R, int lane) {
  const int g = lane >> 2, t = lane & 3;
  float lh[2][4] = {}, hl[2][4] = {};  // separate chains for the lo*hi and hi*lo terms: shorter dependent MMA chains
#pragma unroll
  for (int ks = 0; ks < 2; ++ks) {
    const float af[4] = {lget(g, 8 * ks + t), lget(g + 8, 8 * ks + t), lget(g, 8 * ks + t + 4), lget(g + 8, 8 * ks + t + 4)};
    uint32_t ah[4], al[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) { ah[e] = to_tf32(af[e]); al[e] = to_tf32(af[e] - __uint_as_float(ah[e])); }
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      const float bf[2] = {R[(8 * ks + t) * BLK_LD + 8 * nt + g], R[(8 * ks + t + 4) * BLK_LD + 8 * nt + g]};
      uint32_t bh[2], bl[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) { bh[e] = to_tf32(bf[e]); bl[e] = to_tf32(bf[e] - __uint_as_float(bh[e])); }
      mma_tf32(acc[nt], ah, bh);
      mma_tf32(lh[nt], al, bh);
      mma_tf32(hl[nt], ah, bl);
    }
  }
#pragma unroll
  for (int nt = 0; nt < 2; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[nt][e] += lh[nt][e] + hl[nt][e];
}
// accumulator fragment -> block in shared memory (optionally negated)
__device__ __forceinline__ void block_store(float* __restrict__ dst, const float (&acc)[2][4], int lane, float sign = 1.f) {
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int nt = 0; nt < 2; ++nt) {
    *reinterpret_cast<float2*>(dst + g * BLK_LD + 8 * nt + 2 * t) = make_float2(sign * acc[nt][0], sign * acc[nt][1]);
    *reinterpret_cast<float2*>(dst + (g + 8) * BLK_LD + 8 * nt + 2 * t) = make_float2(sign * acc[nt][2], sign * acc[nt][3]);
  }
}

// bf16 hi + lo images of a pair of fp32 values: hi = round-to-bf16, lo = bf16(x - hi); packed math on the pair
__device__ __forceinline__ void split_pair(float2 x, uint32_t& hi, uint32_t& lo) {
  hi = pack_bf16x2(x.x, x.y);
  const float2 h = make_float2(__uint_as_float(hi << 16), __uint_as_float(hi & 0xffff0000u));
  const float2 l = __ffma2_rn(h, make_float2(-1.f, -1.f), x);
  lo = pack_bf16x2(l.x, l.y);
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Four gated Gram entries f_i kn_j e^{b_i - b_j} acc_j for columns j0..j0+3 (packed fp32 pairs); entry e is kept when
// keep > e, where the caller passes keep = i - j0 for a strictly lower mask and i - j0 + 1 for a lower one.  The
// difference b_i - b_j is formed before the scaling by log2(e), so nearby tokens lose no accuracy to large |b|.
__device__ __forceinline__ void gate4(float (&out)[4], const uint32_t* acc, float bi, float fi, const float* bs_j, const float* kn_j,
                                      int keep) {
  const float4 b4 = *reinterpret_cast<const float4*>(bs_j), k4 = *reinterpret_cast<const float4*>(kn_j);
  const float2 m1 = make_float2(-1.f, -1.f), bi2 = make_float2(bi, bi), fi2 = make_float2(fi, fi);
  const float2 l2e = make_float2(1.4426950408889634f, 1.4426950408889634f);
  const float2 x0 = __fmul2_rn(__ffma2_rn(make_float2(b4.x, b4.y), m1, bi2), l2e);
  const float2 x1 = __fmul2_rn(__ffma2_rn(make_float2(b4.z, b4.w), m1, bi2), l2e);
  const float2 e0 = make_float2(ex2_approx(x0.x), ex2_approx(x0.y)), e1 = make_float2(ex2_approx(x1.x), ex2_approx(x1.y));
  const float2 r0 = __fmul2_rn(__fmul2_rn(fi2, make_float2(__uint_as_float(acc[0]), __uint_as_float(acc[1]))),
                               __fmul2_rn(make_float2(k4.x, k4.y), e0));
  const float2 r1 = __fmul2_rn(__fmul2_rn(fi2, make_float2(__uint_as_float(acc[2]), __uint_as_float(acc[3]))),
                               __fmul2_rn(make_float2(k4.z, k4.w), e1));
  out[0] = keep > 0 ? r0.x : 0.f; out[1] = keep > 1 ? r0.y : 0.f;
  out[2] = keep > 2 ? r1.x : 0.f; out[3] = keep > 3 ? r1.y : 0.f;
}

constexpr int PREP_THREADS = 256;
// Regions are reused as their contents die, which keeps a CTA at 52 KB so that four fit on an SM:
//   PP_KQ  [K_h0 | Q_h0 | K_h1 | Q_h1]   once the Gram MMA is done the Q halves hold the store images of P hi / P lo, then
//                                        the E, E^2, E^3 block scratch, then Tw hi / Tw lo; after the W MMA the whole
//                                        region is the store image of W^T hi | W^T lo
//   PP_R2  A -> T blocks and D^-1 blocks
constexpr int PP_KQ = 0, PP_TWH = PP_KQ + 8192, PP_TWL = PP_KQ + 24576,
              PP_WHI = PP_KQ, PP_WLO = PP_KQ + 16384,
              PP_R2 = 32768, PP_A = PP_R2, PP_DI = PP_A + 10 * BLK_FLOATS * 4,
              PP_SC = PP_R2 + 18432, PP_BARS = PP_SC + 4 * C * 4;
constexpr int PP_PHI = PP_TWH, PP_PLO = PP_TWL;        // P hi / P lo tile images, before the block scratch
constexpr int PP_E = PP_TWH, PP_E2 = PP_TWL, PP_E3 = PP_E2 + 3 * BLK_FLOATS * 4;
static_assert(6 * BLK_FLOATS * 4 <= 8192 && 4 * BLK_FLOATS * 4 <= 8192, "block scratch must fit inside the Q halves");
static_assert(PP_DI + 4 * BLK_FLOATS * 4 <= PP_R2 + 18432, "T and D^-1 blocks must fit inside their region");
constexpr size_t PREP_SMEM = PP_BARS + 64 + 1024;
constexpr uint32_t PT_GRAM = 0, PT_W = 0;               // TMEM columns (64 allocated; W^T reuses the Gram columns)

// Pass 1 per (chunk, value head):
//   tensor cores: [K; Q] K^T                                   -> A (strict lower, gated) and P (lower, gated)
//   CUDA cores  : T = (I + A)^-1 by 16x16 blocks (warp-level tf32 MMAs for the block products)
//   tensor cores: W^T = K^T (T diag(beta e^b))^T   (M = 128 = d_k, N = 64 tokens)
// W^T leaves as bf16 hi + lo, as the 128-byte-swizzled shared-memory image of a [128][64] tile (one bulk copy out here,
// one bulk copy in by the scan, which reads it as an MN-major B operand); Tu = T diag(beta) leaves as bf16 hi + lo
// [64][64] tiles in the same swizzled layout: the scan forms U^T = V^T Tu^T itself, straight into its Vn accumulator.
__global__ void __launch_bounds__(PREP_THREADS, 4)
chunk_prep_kernel(const AveGdnArgs a, const __grid_constant__ GdnMaps maps, const int32_t* __restrict__ chunk_start, PrepOut out,
                  const __grid_constant__ ScanPlan plan, int compact_grid) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  float* Ab = reinterpret_cast<float*>(smem + PP_A);   // A as 16x16 blocks (r >= c), block tri(r,c); later T
  float* Di = reinterpret_cast<float*>(smem + PP_DI);  // (I + A_rr)^-1
  float* Eb = reinterpret_cast<float*>(smem + PP_E);
  float* E2b = reinterpret_cast<float*>(smem + PP_E2);
  float* E3b = reinterpret_cast<float*>(smem + PP_E3);
  float* bs = reinterpret_cast<float*>(smem + PP_SC);
  float* betas = bs + C;
  float* qn = betas + C;
  float* kn = qn + C;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + PP_BARS);
  uint64_t* tma_bar = bars;
  uint64_t* mma_bar = bars + 1;
  uint64_t* mma2_bar = bars + 2;   // W^T accumulated
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int h = blockIdx.y, tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  // Whole-batch launches index every chunk of the batch; range launches use the compact grid
  // n_seqs x parts x rn so that no CTA is spent on chunks outside the range.
  int c = blockIdx.x;
  if (compact_grid) {
    const int per_seq = plan.parts * plan.rn;
    const int n = blockIdx.x / per_seq, rest = blockIdx.x % per_seq;
    const int cis = plan.part_begin[rest / plan.rn] + plan.r0 + rest % plan.rn;
    if (a.cu_seqlens != nullptr && chunk_start[a.n_seqs] < 0) return;  // table rejected
    const int per = a.cu_seqlens ? (chunk_start[n + 1] - chunk_start[n]) : (a.T + C - 1) / C;
    if (cis >= per || cis >= plan.part_begin[rest / plan.rn + 1]) return;
    c = (a.cu_seqlens ? chunk_start[n] : n * per) + cis;
  }
  const ChunkRef cr = find_chunk(a, chunk_start, c);  // (a compact grid only ever names chunks of this launch's range)
  if (!cr.ok) return;
  const int hk = h / (a.Hv / a.Hk);
  const int64_t rec = (int64_t)c * a.Hv + h;

  if (tid == 0) {
    tc::mbar_init(tma_bar, 1);
    tc::mbar_init(mma_bar, 1);
    tc::mbar_init(mma2_bar, 1);
    *abort_flag = 0;
    tc::fence_barrier_init();
    tc::mbar_expect_tx(tma_bar, 32768);
    tc::tma_load_4d(smem + PP_KQ, &maps.k, tma_bar, 0, hk, cr.t0, cr.b);
    tc::tma_load_4d(smem + PP_KQ + 8192, &maps.q, tma_bar, 0, hk, cr.t0, cr.b);
    tc::tma_load_4d(smem + PP_KQ + 16384, &maps.k, tma_bar, 64, hk, cr.t0, cr.b);
    tc::tma_load_4d(smem + PP_KQ + 24576, &maps.q, tma_bar, 64, hk, cr.t0, cr.b);
  }
  if (warp == 2) tc::tmem_alloc(tmem_slot, 64);
  if (tid < C) {
    const bool valid = tid < cr.len;
    const int64_t off = cr.b * a.g_stride_b + (int64_t)(cr.t0 + tid) * a.g_stride_t + h;
    bs[tid] = valid ? a.g[off] : 0.f;
    betas[tid] = valid ? a.beta[off] : 0.f;
  }
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tm = *tmem_slot;
  if (warp == 1) {  // in-chunk cumulative gate: inclusive scan of 64 values by one warp
    float v0 = bs[lane], v1 = bs[32 + lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float t0 = __shfl_up_sync(0xffffffffu, v0, o), t1 = __shfl_up_sync(0xffffffffu, v1, o);
      if (lane >= o) { v0 += t0; v1 += t1; }
    }
    v1 += __shfl_sync(0xffffffffu, v0, 31);
    bs[lane] = v0; bs[32 + lane] = v1;
  }

  // Only warp 0 polls an mbarrier; the other warps park at the next CTA barrier (a hardware barrier costs no issue
  // slots, a polling loop does) and learn of a failed wait through the abort flag.
  bool ok = true;
  if (warp == 0) {
    ok = tc::mbar_wait_warp(tma_bar, 0, abort_flag);
    tc::tc_fence_after_sync();
    const bool leader = tc::elect_one();
    if (ok && leader) {
      constexpr uint32_t idesc = tc::idesc_f16(128, 64, 1, 1, false, false);
      const uint32_t base = tc::smem_u32(smem + PP_KQ);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint64_t d = tc::smem_desc_sw128(base + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024);
        tc::mma_ss(tm + PT_GRAM, d, d, idesc, k != 0 ? 1u : 0u);
      }
      tc::mma_commit(mma_bar);
    }
    __syncwarp();
  }
  // row norms of k and q (the swizzle only permutes 16-byte pieces inside a 128-byte row, so a row sum needs no decode)
  if (a.flags & AVE_GDN_FLAG_QK_L2NORM) {
    __syncthreads();  // warp 0 has seen the tiles land
    const int i = tid >> 2, part = tid & 3;
    float sk = 0.f, sq = 0.f;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const uint4 kr = *reinterpret_cast<const uint4*>(smem + PP_KQ + half * 16384 + i * 128 + part * 32);
      const uint4 kr2 = *reinterpret_cast<const uint4*>(smem + PP_KQ + half * 16384 + i * 128 + part * 32 + 16);
      const uint4 qr = *reinterpret_cast<const uint4*>(smem + PP_KQ + 8192 + half * 16384 + i * 128 + part * 32);
      const uint4 qr2 = *reinterpret_cast<const uint4*>(smem + PP_KQ + 8192 + half * 16384 + i * 128 + part * 32 + 16);
      const uint32_t kw[8] = {kr.x, kr.y, kr.z, kr.w, kr2.x, kr2.y, kr2.z, kr2.w};
      const uint32_t qw[8] = {qr.x, qr.y, qr.z, qr.w, qr2.x, qr2.y, qr2.z, qr2.w};
#pragma unroll
      for (int w = 0; w < 8; ++w) {
        const float k0 = __uint_as_float(kw[w] << 16), k1 = __uint_as_float(kw[w] & 0xffff0000u);
        const float q0 = __uint_as_float(qw[w] << 16), q1 = __uint_as_float(qw[w] & 0xffff0000u);
        sk += k0 * k0 + k1 * k1; sq += q0 * q0 + q1 * q1;
      }
    }
    sk += __shfl_xor_sync(0xffffffffu, sk, 1); sk += __shfl_xor_sync(0xffffffffu, sk, 2);
    sq += __shfl_xor_sync(0xffffffffu, sq, 1); sq += __shfl_xor_sync(0xffffffffu, sq, 2);
    if (part == 0) { kn[i] = rsqrtf(sk + 1e-6f); qn[i] = rsqrtf(sq + 1e-6f); }
  } else if (tid < C) { kn[tid] = 1.f; qn[tid] = 1.f; }
  __syncthreads();
  const float bC = bs[C - 1];
  float* fwv = qn;  // q's norm is consumed below; afterwards the slot holds beta_j e^{b_j} kn_j, the column factor of Tw
  if (tid < C) {
    float* sc = out.scal + rec * SCAL_FLOATS;
    sc[tid] = __expf(bs[tid]) * qn[tid] * a.scale;   // o_i = qs_i (H q_i) + (scale P Vn)_i: the output scale is folded in here and in P
    sc[C + tid] = __expf(bC - bs[tid]) * kn[tid];    // Vd_j = ks_j Vn_j
    sc[2 * C + tid] = __expf(bC);
  }
  if (warp == 0) tc::mbar_wait_warp(mma_bar, 0, abort_flag);
  __syncthreads();
  ok = *abort_flag == 0u;
  tc::tc_fence_after_sync();
  {
    const int quarter = warp & 3, colhalf = warp >> 2;
    const int r = quarter * 32 + lane;
    // warps whose 32 columns all lie above their 32 rows (rows 0..31 against columns 32..63) have nothing to gate
    const bool above = colhalf > (quarter & 1);
    uint32_t acc[32];
    if (!above) {
      tc::tmem_ld32(tm + PT_GRAM + ((uint32_t)(quarter * 32) << 16) + 32 * colhalf, acc);
      tc::tmem_ld_wait();
    }
    if (r < C) {  // A = strict_lower(beta_i e^{b_i-b_j} k_i.k_j); blocks above the diagonal are not stored
      const int i = r;
      const float bi = bs[i], fi = betas[i] * kn[i];
      if (!above) {
#pragma unroll
        for (int j4 = 0; j4 < 8; ++j4) {
          const int j0 = 32 * colhalf + 4 * j4;
          float av[4];
          gate4(av, acc + 4 * j4, bi, fi, bs + j0, kn + j0, i - j0);
          if ((j0 >> 4) <= (i >> 4))
            *reinterpret_cast<float4*>(Ab + tri(i >> 4, j0 >> 4) * BLK_FLOATS + (i & 15) * BLK_LD + (j0 & 15)) =
                make_float4(av[0], av[1], av[2], av[3]);
        }
      }
    } else {      // P = lower_incl(e^{b_i-b_j} q_i.k_j), bf16 hi + lo
      const int i = r - C;
      const float bi = bs[i], fi = (i < cr.len) ? qn[i] * a.scale : 0.f;
      uint32_t ph[16], pl[16];
      if (!above) {
#pragma unroll
        for (int j4 = 0; j4 < 8; ++j4) {
          const int j0 = 32 * colhalf + 4 * j4;
          float pv[4];
          gate4(pv, acc + 4 * j4, bi, fi, bs + j0, kn + j0, i - j0 + 1);
          split_pair(make_float2(pv[0], pv[1]), ph[2 * j4], pl[2 * j4]);
          split_pair(make_float2(pv[2], pv[3]), ph[2 * j4 + 1], pl[2 * j4 + 1]);
        }
      } else {
#pragma unroll
        for (int w = 0; w < 16; ++w) { ph[w] = 0u; pl[w] = 0u; }
      }
      // the Q halves are dead (the Gram MMA is complete): they take the swizzled tile images of P hi and P lo, which
      // leave with one bulk copy each
      uint4* ih = reinterpret_cast<uint4*>(smem + PP_PHI + i * 128);
      uint4* il = reinterpret_cast<uint4*>(smem + PP_PLO + i * 128);
#pragma unroll
      for (int v4 = 0; v4 < 4; ++v4) {
        const int piece = (4 * colhalf + v4) ^ (i & 7);
        ih[piece] = make_uint4(ph[4 * v4], ph[4 * v4 + 1], ph[4 * v4 + 2], ph[4 * v4 + 3]);
        il[piece] = make_uint4(pl[4 * v4], pl[4 * v4 + 1], pl[4 * v4 + 2], pl[4 * v4 + 3]);
      }
      tc::fence_proxy_async_smem();
    }
  }
  __syncthreads();
  if (tid == 0 && ok) {
    tc::bulk_store(out.p_hi + rec * (C * C), smem + PP_PHI, REC_P);
    tc::bulk_store(out.p_lo + rec * (C * C), smem + PP_PLO, REC_P);
    tc::bulk_commit();
  }
  // ---- T = (I + A)^-1 by 16x16 blocks.  With D = blockdiag(I + A_rr) and E = D^-1 (A - A_D) (strictly block lower,
  // E^4 = 0):  T = (I - E + E^2 - E^3) D^-1.  Only the four small D_r^-1 need a sequential substitution.
  if (tid < 64) {  // column k of (I + A_rr)^-1, 16 rows, one thread each
    const int r = tid >> 4, k = tid & 15;
    const float* Arr = Ab + tri(r, r) * BLK_FLOATS;
    float x[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      float s0 = (i == k) ? 1.f : 0.f, s1 = 0.f;
#pragma unroll
      for (int j = 0; j < i; ++j) {
        const float av = Arr[i * BLK_LD + j];
        if (j & 1) s1 = fmaf(-av, x[j], s1); else s0 = fmaf(-av, x[j], s0);
      }
      x[i] = s0 + s1;
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) Di[r * BLK_FLOATS + i * BLK_LD + k] = x[i];
  } else if (tid < 128) {  // q's norms are no longer read: reuse their slot for the column factors of Tw
    const int j = tid - 64;
    fwv[j] = betas[j] * __expf(bs[j]) * kn[j];
  }
  if (tid == 0) tc::bulk_wait_read<0>();  // the P images have been read: the block scratch may overwrite them
  __syncthreads();
  // E_rc = D_r^-1 A_rc, r > c: six products, one warp each
  if (warp < 6) {
    constexpr int RR[6] = {1, 2, 2, 3, 3, 3}, CC[6] = {0, 0, 1, 0, 1, 2};
    const int r = RR[warp], c = CC[warp];
    float acc[2][4] = {};
    const float* L = Di + r * BLK_FLOATS;
    block_mma(acc, [&](int row, int col) { return L[row * BLK_LD + col]; }, Ab + tri(r, c) * BLK_FLOATS, lane);
    block_store(Eb + (tri(r, c) - r) * BLK_FLOATS, acc, lane);  // strictly-lower block index: tri(r,c) - r
  }
  __syncthreads();
  // E^2: (2,0) = E21 E10, (3,1) = E32 E21, (3,0) = E31 E10 + E32 E20
  auto Eblk = [&](int r, int c) { return Eb + (tri(r, c) - r) * BLK_FLOATS; };
  if (warp < 3) {
    float acc[2][4] = {};
    if (warp == 0) {
      const float* L = Eblk(2, 1);
      block_mma(acc, [&](int row, int col) { return L[row * BLK_LD + col]; }, Eblk(1, 0), lane);
    } else if (warp == 1) {
      const float* L = Eblk(3, 2);
      block_mma(acc, [&](int row, int col) { return L[row * BLK_LD + col]; }, Eblk(2, 1), lane);
    } else {
      const float* L1 = Eblk(3, 1);
      block_mma(acc, [&](int row, int col) { return L1[row * BLK_LD + col]; }, Eblk(1, 0), lane);
      const float* L2 = Eblk(3, 2);
      block_mma(acc, [&](int row, int col) { return L2[row * BLK_LD + col]; }, Eblk(2, 0), lane);
    }
    block_store(E2b + warp * BLK_FLOATS, acc, lane);  // order: (2,0), (3,1), (3,0)
  }
  __syncthreads();
  // E^3: (3,0) = E32 E2_20
  if (warp == 0) {
    float acc[2][4] = {};
    const float* L = Eblk(3, 2);
    block_mma(acc, [&](int row, int col) { return L[row * BLK_LD + col]; }, E2b, lane);
    block_store(E3b, acc, lane);
  }
  __syncthreads();
  // T_rc = (-E + E^2 - E^3)_rc D_c^-1, r > c (written over A_rc, which is no longer needed); T_rr = D_r^-1
  if (warp < 6) {
    constexpr int RR[6] = {1, 2, 2, 3, 3, 3}, CC[6] = {0, 0, 1, 0, 1, 2};
    const int r = RR[warp], c = CC[warp];
    const float* e1 = Eblk(r, c);
    const float* e2 = (r - c >= 2) ? E2b + ((r == 2) ? 0 : (c == 1 ? 1 : 2)) * BLK_FLOATS : nullptr;
    const float* e3 = (r - c == 3) ? E3b : nullptr;
    float acc[2][4] = {};
    block_mma(acc, [&](int row, int col) {
      float v = -e1[row * BLK_LD + col];
      if (e2 != nullptr) v += e2[row * BLK_LD + col];
      if (e3 != nullptr) v -= e3[row * BLK_LD + col];
      return v;
    }, Di + c * BLK_FLOATS, lane);
    block_store(Ab + tri(r, c) * BLK_FLOATS, acc, lane);
  }
  __syncthreads();
  // Tw = T diag(beta e^b kn) as bf16 hi + lo K-major tiles [i][j] with the 128-byte swizzle (B operand of the W MMA);
  // Tu = T diag(beta) as bf16 hi + lo straight to scratch, in the same swizzled tile layout (the scan brings it in with
  // a bulk copy).  A thread owns one 16-byte piece (8 columns) of two rows; a warp covers four full rows per store.
  {
    const int pc = tid & 7, cb = pc >> 1;
    float fw[8], fu[8];
    {
      const float4 a0 = *reinterpret_cast<const float4*>(fwv + 8 * pc), a1 = *reinterpret_cast<const float4*>(fwv + 8 * pc + 4);
      const float4 b0 = *reinterpret_cast<const float4*>(betas + 8 * pc), b1 = *reinterpret_cast<const float4*>(betas + 8 * pc + 4);
      fw[0] = a0.x; fw[1] = a0.y; fw[2] = a0.z; fw[3] = a0.w; fw[4] = a1.x; fw[5] = a1.y; fw[6] = a1.z; fw[7] = a1.w;
      fu[0] = b0.x; fu[1] = b0.y; fu[2] = b0.z; fu[3] = b0.w; fu[4] = b1.x; fu[5] = b1.y; fu[6] = b1.z; fu[7] = b1.w;
    }
    uint4* guh = reinterpret_cast<uint4*>(out.tu_hi + rec * (C * C));
    uint4* gul = reinterpret_cast<uint4*>(out.tu_lo + rec * (C * C));
#pragma unroll
    for (int it = 0; it < 2; ++it) {
      const int i = (tid >> 3) + 32 * it, rb = i >> 4;
      float t[8];
      if (cb <= rb) {
        const float* src = ((rb == cb) ? Di + rb * BLK_FLOATS : Ab + tri(rb, cb) * BLK_FLOATS) + (i & 15) * BLK_LD + (pc & 1) * 8;
        const float4 t0 = *reinterpret_cast<const float4*>(src), t1 = *reinterpret_cast<const float4*>(src + 4);
        t[0] = t0.x; t[1] = t0.y; t[2] = t0.z; t[3] = t0.w; t[4] = t1.x; t[5] = t1.y; t[6] = t1.z; t[7] = t1.w;
#pragma unroll
        for (int e = 0; e < 8; ++e) t[e] = (8 * pc + e <= i) ? t[e] : 0.f;
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) t[e] = 0.f;
      }
      uint32_t wh[4], wl[4], uh[4], ul[4];
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float2 tp = make_float2(t[2 * w], t[2 * w + 1]);
        split_pair(__fmul2_rn(tp, make_float2(fw[2 * w], fw[2 * w + 1])), wh[w], wl[w]);
        split_pair(__fmul2_rn(tp, make_float2(fu[2 * w], fu[2 * w + 1])), uh[w], ul[w]);
      }
      const uint32_t off = (uint32_t)(i * 128 + ((pc ^ (i & 7)) << 4));
      *reinterpret_cast<uint4*>(smem + PP_TWH + off) = make_uint4(wh[0], wh[1], wh[2], wh[3]);
      *reinterpret_cast<uint4*>(smem + PP_TWL + off) = make_uint4(wl[0], wl[1], wl[2], wl[3]);
      if (ok) {
        guh[i * 8 + (pc ^ (i & 7))] = make_uint4(uh[0], uh[1], uh[2], uh[3]);  // same swizzled image as in shared memory
        gul[i * 8 + (pc ^ (i & 7))] = make_uint4(ul[0], ul[1], ul[2], ul[3]);
      }
    }
  }
  tc::fence_proxy_async_smem();
  __syncthreads();
  constexpr uint32_t idesc_w = tc::idesc_f16(128, 64, 1, 1, true, false);  // A MN-major (token rows), B K-major
  if (warp == 0) {
    const bool leader = tc::elect_one();
    if (ok && leader) {
      const uint32_t kbase = tc::smem_u32(smem + PP_KQ);
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        const uint32_t tw = tc::smem_u32(smem + (t ? PP_TWL : PP_TWH));
#pragma unroll
        for (int k = 0; k < 4; ++k)  // K halves sit 16384 bytes apart (the Q halves' slots lie between them)
          tc::mma_ss(tm + PT_W, tc::smem_desc_sw128(kbase + k * 2048, 16384, 1024), tc::smem_desc_sw128(tw + k * 32, 16, 1024), idesc_w,
                     (t | k) != 0 ? 1u : 0u);
      }
      tc::mma_commit(mma2_bar);
    }
    __syncwarp();
  }
  if (warp == 0) tc::mbar_wait_warp(mma2_bar, 0, abort_flag);
  __syncthreads();
  ok = ok && *abort_flag == 0u;
  tc::tc_fence_after_sync();
  {
    // Each lane owns one row of W^T (a d_k index) and each warp half of its 64 tokens.  The K, Q and Tw tiles are dead
    // now; the bf16 hi and lo rows are written over them in the 128-byte-swizzled tile layout the scan's MMA reads, so
    // that the tile leaves with one bulk copy and arrives in the scan's shared memory with another, unchanged.
    const int quarter = warp & 3, colhalf = warp >> 2;
    const int r = quarter * 32 + lane;
    uint32_t acc[32];
    tc::tmem_ld32(tm + PT_W + ((uint32_t)(quarter * 32) << 16) + 32 * colhalf, acc);
    tc::tmem_ld_wait();
    uint4* ih = reinterpret_cast<uint4*>(smem + PP_WHI + r * 128);
    uint4* il = reinterpret_cast<uint4*>(smem + PP_WLO + r * 128);
#pragma unroll
    for (int p4 = 0; p4 < 4; ++p4) {
      uint32_t hi[4], lo[4];
#pragma unroll
      for (int w = 0; w < 4; ++w)
        split_pair(make_float2(__uint_as_float(acc[8 * p4 + 2 * w]), __uint_as_float(acc[8 * p4 + 2 * w + 1])), hi[w], lo[w]);
      const int piece = (4 * colhalf + p4) ^ (r & 7);
      ih[piece] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
      il[piece] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    }
  }
  tc::fence_proxy_async_smem();
  tc::tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && ok) {
    tc::bulk_store(out.w_hi + rec * (C * D), smem + PP_WHI, REC_W);
    tc::bulk_store(out.w_lo + rec * (C * D), smem + PP_WLO, REC_W);
    tc::bulk_commit();
    tc::bulk_wait_read<0>();  // shared memory must stay intact until the copies have read it
  }
  if (warp == 2) {
    tc::tc_fence_after_sync();
    tc::tmem_dealloc(tm, 64);
  }
  if (!ok && tid == 0 && a.status != nullptr) atomicOr(a.status, AVE_GDN_DEV_WAIT_EXPIRED);
}

// ------------------------------------------------------------------------------------------------ pass 2
// Warpgroup 0: warp 0 loader, warps 1 and 2 MMA issuers; warpgroups 1..NG: chain epilogue, each covering all 128 TMEM
// lanes and 1/NG of the columns; the last warpgroup: output.  (Four epilogue groups at 80 registers were measured: no
// faster, the epilogue is bound by the instructions issued per scheduler, not by the work per thread.)
constexpr int NG = 2;
constexpr int SCAN_THREADS = 32 * (4 + 4 * NG + 4);
constexpr int REGS_LAUNCH = 128;
constexpr int REGS_CTRL = 72, REGS_CHAIN = 168, REGS_OUT = 104;
static_assert(NG == 2, "the register split below is for two epilogue groups");
static_assert(REGS_CTRL + NG * REGS_CHAIN + REGS_OUT <= (NG + 2) * REGS_LAUNCH, "register redistribution exceeds the launch allocation");
static_assert(SCAN_THREADS * REGS_LAUNCH <= 65536, "launch allocation exceeds the register file");
constexpr int HC = D / NG;   // columns of H (d_k) per chain-epilogue group
constexpr int VC = C / NG;   // columns of Vn (tokens) per group
constexpr int ST_WHI = 0, ST_WLO = 16384, ST_Q = 32768, ST_K = 49152, ST_PHI = 65536, ST_PLO = 73728, ST_V = 81920;
constexpr int STAGE = 98304;                         // multiple of 1024
constexpr int SCAL_BYTES = SCAL_FLOATS * 4;
constexpr uint32_t TILES_TX = STAGE - 2 * REC_P;  // W hi, W lo, Q, K, V
constexpr int OFF_SCAL = 2 * STAGE;                  // 4 x [qs | ks | decay]: a deeper ring than the tile stages, because
                                                     // the output warps read qs up to a chunk after the stage is recycled
constexpr int OFF_VT = OFF_SCAL + 4 * SCAL_BYTES;    // single buffer: Tu hi | Tu lo (they come from scratch that pass 1 has
                                                     // just written; the V tile, an input read with a long-latency strided
                                                     // pattern, rides in the stage ring a chunk ahead)
constexpr int VT_TUH = 0, VT_TUL = 8192, VT_BYTES = 16384;
static_assert(OFF_VT % 1024 == 0, "swizzled tiles need 1024-byte alignment");
constexpr int OFF_BARS = OFF_VT + VT_BYTES;
constexpr size_t SCAN_SMEM = OFF_BARS + 256 + 1024;
// TMEM columns
constexpr uint32_t TM_HHI = 0, TM_HLO = 64, TM_VN = 128, TM_VNHI = 192, TM_VNLO = 224, TM_O1 = 256, TM_O2 = 320, TM_DH = 384;
// The bf16 hi and lo images of Vd reuse the Vn accumulator's columns.  Each chain-epilogue group packs its VC tokens
// into its own VC columns (hi in the first half, lo in the second), so a warp overwrites only columns it has itself
// read and the groups need no barrier between reading the accumulator and writing the images.  Their only reader is
// the state-increment MMA, issued by the same thread that next writes the accumulator (U^T of the following chunk),
// so program order protects them.  (The images of Vn, read by the other issuer's O2, have columns of their own.)
// 16-token K step k of the Vd image starts at:
__host__ __device__ constexpr uint32_t vd_img_col(int k, bool lo) {
  return TM_VN + (uint32_t)(VC * ((16 * k) / VC) + ((16 * k) % VC) / 2 + (lo ? VC / 2 : 0));
}

// Issues `ksteps` MMAs D (+)= A[tmem] * B[smem] over consecutive 16-wide K steps.  A advances 8 TMEM columns per
// step; B advances b_step bytes per step and jumps b_half extra after four steps (second 64-wide K half of a
// K-major tile; 0 when there is none).
__device__ __forceinline__ void issue_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_smem, uint32_t b_step, uint32_t b_half,
                                         uint32_t lbo, uint32_t idesc, int ksteps, bool accumulate) {
  const uint64_t desc = tc::smem_desc_sw128(b_smem, lbo, 1024);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    if (k < ksteps)
      tc::mma_ts(d_tmem, a_tmem + 8 * k, desc + (uint64_t)((k * b_step + ((k > 3) ? b_half : 0u)) >> 4), idesc,
                 (accumulate || k != 0) ? 1u : 0u);
  }
}

// kMulti: built with the parallel-parts machinery (ScanPlan::parts > 1).  The plain instantiation carries none of its
// state, which keeps the output warpgroup inside its register budget with 32-token pieces.
template <bool kMulti>
__global__ void __launch_bounds__(SCAN_THREADS, 1)
chunk_scan_tc_kernel(const AveGdnArgs a, const __grid_constant__ GdnMaps maps, const int32_t* __restrict__ chunk_start,
                     const __nv_bfloat16* __restrict__ w_hi_ws, const __nv_bfloat16* __restrict__ w_lo_ws,
                     const __nv_bfloat16* __restrict__ p_hi_ws, const __nv_bfloat16* __restrict__ p_lo_ws,
                     const __nv_bfloat16* __restrict__ tu_hi_ws, const __nv_bfloat16* __restrict__ tu_lo_ws,
                     const float* __restrict__ scal_ws, float* __restrict__ o_f32, uint8_t* __restrict__ qt_img,
                     float* __restrict__ carry, uint8_t* __restrict__ m0_pack, const int32_t* __restrict__ seq_order,
                     const __grid_constant__ ScanPlan plan) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BARS);
  uint64_t* full = bars;          // [2] W, Q, K and V tiles of the stage landed
  uint64_t* pfull = bars + 2;     // [2] P tiles and the scale vectors of the stage landed
  uint64_t* h_ready = bars + 4;   // bf16 image of the state is in TMEM
  uint64_t* vn_full = bars + 5;   // -(H W^T) accumulated
  uint64_t* vn_ready = bars + 6;  // Vn / Vd hi+lo written back to TMEM
  uint64_t* dh_full = bars + 7;   // state increment accumulated
  uint64_t* o_full = bars + 8;    // both output accumulators complete
  uint64_t* o1_empty = bars + 9;  // O1 accumulator drained (the output warps take it first, whole, so O1 of the next chunk can run early)
  uint64_t* o2_empty = bars + 12; // O2 accumulator drained
  uint64_t* o1_done = bars + 13;  // O1 complete: the bf16 image of H may be overwritten
  uint64_t* u_full = bars + 10;   // Tu tiles landed
  uint64_t* u_empty = bars + 11;  // the U^T MMAs that read them are complete
  uint64_t* vd_ready = bars + 14; // Vd hi+lo written to TMEM (the state update needs nothing else)
  // a stage is given back tile by tile, as soon as the last MMA that reads the tile is complete
  uint64_t* w_empty = bars + 16;  // [2] after the Vn MMAs
  uint64_t* q_empty = bars + 18;  // [2] after O1
  uint64_t* k_empty = bars + 20;  // [2] after the state increment
  uint64_t* p_empty = bars + 22;  // [2] after O2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // One CTA per (sequence, chain, value head).  Chain 0 is part 0; chains 2p-1 and 2p are the local and the transition
  // chain of part p >= 1 (see ScanPlan).
  const int chains = kMulti ? 2 * plan.parts - 1 : 1;
  const int h = blockIdx.x % a.Hv;
  const int unit = blockIdx.x / a.Hv;
  const int chain = kMulti ? unit % chains : 0;
  const int n = seq_order ? seq_order[unit / chains] : unit / chains;  // varlen: longest sequences first
  const int part = (chain + 1) >> 1;
  const bool phi = kMulti && chain > 0 && (chain & 1) == 0;
  const int hk = h / (a.Hv / a.Hk);
  if (a.cu_seqlens != nullptr && chunk_start[a.n_seqs] < 0) return;  // the chunk table was rejected: nothing runs
  SeqSpan sp = seq_span(a.cu_seqlens, n, a.T, a.status);
  // longer than the caller's bound: the launch schedule was sized from that bound, so the sequence is skipped (zero
  // output, no state access, like a negative slot) and flagged
  const bool too_long = a.cu_seqlens != nullptr && a.max_seqlen > 0 && sp.len > a.max_seqlen;
  if (too_long && a.status != nullptr && threadIdx.x == 0) atomicOr(a.status, AVE_GDN_DEV_BAD_SEQLEN);
  if (!sp.ok || sp.len == 0) {
    if (plan.r0 > 0 || chain > 0) return;
    // zero-length sequence: the final state is the initial state
    if (sp.ok && a.final_state != nullptr && a.final_state != a.initial_state) {
      const int slot0 = a.state_indices ? a.state_indices[n] : n;
      if (slot0 >= 0 && slot0 < a.num_slots) {
        const int64_t tile0 = ((int64_t)slot0 * a.Hv + h) * (int64_t)(D * D);
        for (int e = threadIdx.x; e < D * D; e += SCAN_THREADS)
          a.final_state[tile0 + e] = a.initial_state ? a.initial_state[tile0 + e] : 0.f;
      }
    }
    return;
  }
  const int seq_chunks = (sp.len + C - 1) / C;
  // a sequence that ends inside part 0 is one plain chain: outputs and the final state leave directly
  const bool multi = kMulti && plan.parts > 1 && seq_chunks > plan.part_begin[1] && !too_long;
  if (chain > 0 && (!multi || plan.part_begin[part] >= seq_chunks)) return;
  int slot = n;
  if (a.state_indices != nullptr) {
    slot = a.state_indices[n];
    if (slot >= a.num_slots) {
      if (a.status != nullptr && threadIdx.x == 0) atomicOr(a.status, AVE_GDN_DEV_BAD_SLOT);
      slot = -1;
    }
  }
  if (too_long) slot = -1;
  __nv_bfloat16* og = reinterpret_cast<__nv_bfloat16*>(a.o) + sp.b * a.o_stride_b + (int64_t)h * a.o_stride_h;
  // where this chain's per-token rows go: the local rows of later parts wait in fp32 scratch for the fix-up; part 0
  // writes fp32 scratch only when a gated norm follows, else the result itself; the transition chain's rows leave as
  // the bf16 hi/lo operand images the fix-up's MMAs read (see the output warps)
  float* const out_f32 = (!phi && (a.z != nullptr || part > 0)) ? o_f32 : nullptr;
  if (slot < 0) {  // skipped sequence: zero output, no state access (chain 0 clears the whole sequence once)
    if (chain > 0 || plan.r0 > 0) return;
    float* zf = a.z != nullptr ? o_f32 : nullptr;
    for (int e = threadIdx.x; e < sp.len * D; e += SCAN_THREADS) {
      const int64_t tok = sp.t0 + e / D;
      if (zf != nullptr) zf[(((int64_t)sp.b * a.T + tok) * a.Hv + h) * D + e % D] = 0.f;
      else og[tok * a.o_stride_t + e % D] = __float2bfloat16(0.f);
    }
    return;
  }
  // This launch covers chunks [c_lo, c_hi) of the chain's part; the state enters from / leaves to the carry buffer
  // unless this is the first / last launch of a plain chain.
  const int part_end = min(plan.part_begin[part + 1], seq_chunks);
  const int c_lo = plan.part_begin[part] + plan.r0;
  const int c_hi = min(c_lo + plan.rn, part_end);
  if (c_lo >= c_hi) return;  // finished in an earlier launch, or not reached yet
  const bool seg_first = plan.r0 == 0;
  const bool seg_last = c_hi == part_end && !multi;
  const int c_first = (a.cu_seqlens ? chunk_start[n] : n * ((a.T + C - 1) / C)) + c_lo;
  sp.t0 += c_lo * C;
  sp.len = min(sp.len - c_lo * C, (c_hi - c_lo) * C);
  const int n_chunks = c_hi - c_lo;
  const int64_t carry_tile = (((int64_t)n * chains + chain) * a.Hv + h) * (int64_t)(D * D);

  if (threadIdx.x == 0) {
    tc::mbar_init(&full[0], 1); tc::mbar_init(&full[1], 1);
    tc::mbar_init(&pfull[0], 1); tc::mbar_init(&pfull[1], 1);
    for (int i = 0; i < 2; ++i) { tc::mbar_init(&w_empty[i], 1); tc::mbar_init(&q_empty[i], 1); tc::mbar_init(&k_empty[i], 1); tc::mbar_init(&p_empty[i], 1); }
    tc::mbar_init(h_ready, 4 * NG); tc::mbar_init(vn_full, 1); tc::mbar_init(vn_ready, 4 * NG);
    tc::mbar_init(dh_full, 1); tc::mbar_init(o_full, 1); tc::mbar_init(o1_empty, 4); tc::mbar_init(o2_empty, 4); tc::mbar_init(o1_done, 1);
    tc::mbar_init(u_full, 1); tc::mbar_init(u_empty, 1);
    tc::mbar_init(vd_ready, 4 * NG);
    *abort_flag = 0;
    tc::fence_barrier_init();
  }
  if (warp == 1) tc::tmem_alloc(tmem_slot, 512);
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tm = *tmem_slot;

  if (warp < 4) {
  tc::reg_set<REGS_CTRL, REGS_LAUNCH>();
  if (warp == 0) {
    // ------------------------------------------------------------------ loader
    // Two stages of {W hi, W lo, Q, K, P hi, P lo, V}.  A tile of chunk c+2 is fetched as soon as the last MMA that
    // reads the same tile of chunk c is complete (W after the Vn MMAs, early in the chunk's period; P last), so most of a
    // stage lands more than a period before it is needed instead of a fraction of one.
    if (lane == 0) {
      for (int c = 0; c < n_chunks; ++c) {
        const int s = c & 1;
        const uint32_t free_par = ((uint32_t)(c >> 1) & 1u) ^ 1u;  // parity of "chunk c-2 is done with it"
        uint8_t* st = smem + s * STAGE;
        const int64_t rec = (int64_t)(c_first + c) * a.Hv + h;
        const int tok = sp.t0 + c * C;
        // The Vn MMAs of chunk c-2 are complete: so are its U^T MMAs, issued before them (W and V slots are free), and
        // the MMA warp has long passed its wait for the stage's previous phase, so the barrier can be armed again.
        if (!tc::mbar_wait(&w_empty[s], free_par, abort_flag)) break;
        tc::mbar_expect_tx(&full[s], phi ? TILES_TX - 16384u : TILES_TX);  // the transition chain has no V
        if (!phi) {
          tc::tma_load_4d(st + ST_V, &maps.v, &full[s], 0, h, tok, sp.b);
          tc::tma_load_4d(st + ST_V + 8192, &maps.v, &full[s], 64, h, tok, sp.b);
        }
        tc::bulk_load(st + ST_WHI, w_hi_ws + rec * (C * D), REC_W, &full[s]);  // W^T tile images: 128 d_k rows of 64 tokens
        tc::bulk_load(st + ST_WLO, w_lo_ws + rec * (C * D), REC_W, &full[s]);
        if (!tc::mbar_wait(&q_empty[s], free_par, abort_flag)) break;
        tc::tma_load_4d(st + ST_Q, &maps.q, &full[s], 0, hk, tok, sp.b);
        tc::tma_load_4d(st + ST_Q + 8192, &maps.q, &full[s], 64, hk, tok, sp.b);
        if (!tc::mbar_wait(&k_empty[s], free_par, abort_flag)) break;
        tc::tma_load_4d(st + ST_K, &maps.k, &full[s], 0, hk, tok, sp.b);
        tc::tma_load_4d(st + ST_K + 8192, &maps.k, &full[s], 64, hk, tok, sp.b);
        // P and the scale vectors last.  The scale-vector ring is four deep: the output warps read qs of chunk c-4 until
        // they release its accumulators, which O1 of chunk c-2, and so this wait, comes after.
        if (!tc::mbar_wait(&p_empty[s], free_par, abort_flag)) break;
        tc::mbar_expect_tx(&pfull[s], 2 * REC_P + SCAL_BYTES);
        tc::bulk_load(st + ST_PHI, p_hi_ws + rec * (C * C), REC_P, &pfull[s]);
        tc::bulk_load(st + ST_PLO, p_lo_ws + rec * (C * C), REC_P, &pfull[s]);
        tc::bulk_load(smem + OFF_SCAL + (c & 3) * SCAL_BYTES, scal_ws + rec * SCAL_FLOATS, SCAL_BYTES, &pfull[s]);
        if (phi) continue;
        // Tu of chunk c replaces that of chunk c-1 once the U^T MMAs of chunk c-1 have read it
        if (!tc::mbar_wait(u_empty, ((uint32_t)c & 1u) ^ 1u, abort_flag)) break;
        uint8_t* vt = smem + OFF_VT;
        tc::mbar_expect_tx(u_full, VT_BYTES);
        tc::bulk_load(vt + VT_TUH, tu_hi_ws + rec * (C * C), REC_P, u_full);
        tc::bulk_load(vt + VT_TUL, tu_lo_ws + rec * (C * C), REC_P, u_full);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ chain MMA issuer (whole warp runs the loop, one
    // elected lane issues): the MMAs the recurrence waits for.  One thread needs 20 to 60 cycles per MMA instruction, so
    // the 68 instructions of a chunk are shared between two warps; this one keeps the state-dependent ones short:
    //   U^T(c+1) -> [state published] Vn^T(c) -> [Vd written] dH(c)
    constexpr uint32_t id_vn = tc::idesc_f16(128, 64, 1, 1, false, true, true, false);    // negated A, B = W^T read MN-major
    constexpr uint32_t id_dh = tc::idesc_f16(128, 128, 1, 1, false, true);                // B MN-major
    constexpr uint32_t id_u = tc::idesc_f16(128, 64, 1, 1, true, false);                  // A = V tile read MN-major
    const uint32_t vtb = tc::smem_u32(smem + OFF_VT);
    // U^T = V^T (Tu_hi + Tu_lo)^T opens the Vn^T accumulator of a chunk.  It does not depend on the state, so it is
    // issued a chunk ahead, right behind the previous chunk's state-increment MMAs (which read the Vd images in the
    // same columns and, issued earlier by this thread, complete first): the tensor pipe runs it while the chain
    // epilogue re-packs H.
    auto issue_u = [&](int c) {
      if (phi) return;  // v = 0: U^T = 0, the first Vn MMA overwrites the accumulator instead
      const uint32_t vb = tc::smem_u32(smem + (c & 1) * STAGE + ST_V);
      if (tc::elect_one()) {
#pragma unroll
        for (int t = 0; t < 2; ++t)
#pragma unroll
          for (int k = 0; k < 4; ++k)  // 16 tokens per step: V rows 2048 bytes apart, feature halves 8192 bytes apart
            tc::mma_ss(tm + TM_VN, tc::smem_desc_sw128(vb + k * 2048, 8192, 1024),
                       tc::smem_desc_sw128(vtb + (t ? VT_TUL : VT_TUH) + k * 32, 16, 1024), id_u, (t | k) != 0 ? 1u : 0u);
        tc::mma_commit(u_empty);
      }
      __syncwarp();
    };
    bool issuing = n_chunks > 0 && tc::mbar_wait_warp(&full[0], 0u, abort_flag) && (phi || tc::mbar_wait_warp(u_full, 0u, abort_flag));
    if (issuing) { tc::tc_fence_after_sync(); issue_u(0); }
    for (int c = 0; c < n_chunks && issuing; ++c) {
      const int s = c & 1;
      const uint32_t cp = (uint32_t)c & 1u;
      const uint32_t sb = tc::smem_u32(smem + s * STAGE);  // W, K have landed: this warp waited for the stage a chunk ago
      if (!tc::mbar_wait_warp(h_ready, cp, abort_flag)) break;
      tc::tc_fence_after_sync();
      if (tc::elect_one()) {
        // Vn^T += -(Hhi Whi^T + Hhi Wlo^T + Hlo Whi^T); W^T is one [128 d_k][64 token] tile, 16 d_k rows per step
        issue_ts(tm + TM_VN, tm + TM_HHI, sb + ST_WHI, 2048, 0, 16, id_vn, 8, !phi);
        issue_ts(tm + TM_VN, tm + TM_HHI, sb + ST_WLO, 2048, 0, 16, id_vn, 8, true);
        issue_ts(tm + TM_VN, tm + TM_HLO, sb + ST_WHI, 2048, 0, 16, id_vn, 8, true);
        tc::mma_commit(vn_full);
        tc::mma_commit(&w_empty[s]);
      }
      __syncwarp();
      if (!tc::mbar_wait_warp(vd_ready, cp, abort_flag)) break;
      tc::tc_fence_after_sync();
      if (tc::elect_one()) {
        // dH = (Vd_hi + Vd_lo) contracted with K over the chunk's tokens (K tile read MN-major: 16 token rows per step)
        const uint64_t k_desc = tc::smem_desc_sw128(sb + ST_K, 8192, 1024);
#pragma unroll
        for (int k = 0; k < 4; ++k) tc::mma_ts(tm + TM_DH, tm + vd_img_col(k, false), k_desc + (uint64_t)(128 * k), id_dh, k != 0 ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < 4; ++k) tc::mma_ts(tm + TM_DH, tm + vd_img_col(k, true), k_desc + (uint64_t)(128 * k), id_dh, 1u);
        tc::mma_commit(dh_full);
        tc::mma_commit(&k_empty[s]);
      }
      __syncwarp();
      if (c + 1 < n_chunks) {
        // the next chunk's tiles, polled together so that the latencies of phases that are already complete overlap
        uint64_t* b_f = &full[(c + 1) & 1];
        const uint32_t p_f = (uint32_t)((c + 1) >> 1) & 1u;
        if (!(phi ? tc::mbar_wait_warp(b_f, p_f, abort_flag) : tc::mbar_wait2(b_f, p_f, u_full, (uint32_t)(c + 1) & 1u, abort_flag))) break;
        tc::tc_fence_after_sync();
        issue_u(c + 1);
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------------ output MMA issuer: O1 = H Q^T once the Vn MMAs are
    // complete (so that it runs behind them, while the chain epilogue converts Vn), O2 = Vn P^T once Vn hi/lo are back
    constexpr uint32_t id_n64 = tc::idesc_f16(128, 64, 1, 1, false, false);
    for (int c = 0; c < n_chunks; ++c) {
      const int s = c & 1;
      const uint32_t cp = (uint32_t)c & 1u, u = (uint32_t)(c >> 1);
      const uint32_t sb = tc::smem_u32(smem + s * STAGE);
      if (!tc::mbar_wait3(vn_full, cp, o1_empty, cp ^ 1u, &full[s], u & 1u, abort_flag)) break;
      tc::tc_fence_after_sync();
      if (tc::elect_one()) {
        // O1 = (Hhi + Hlo) Q^T; the chain epilogue waits for its completion before it overwrites the bf16 image of H
        issue_ts(tm + TM_O1, tm + TM_HHI, sb + ST_Q, 32, 8192 - 128, 16, id_n64, 8, false);
        issue_ts(tm + TM_O1, tm + TM_HLO, sb + ST_Q, 32, 8192 - 128, 16, id_n64, 8, true);
        tc::mma_commit(o1_done);
        tc::mma_commit(&q_empty[s]);
      }
      __syncwarp();
      if (!tc::mbar_wait3(vn_ready, cp, o2_empty, cp ^ 1u, &pfull[s], u & 1u, abort_flag)) break;
      tc::tc_fence_after_sync();
      if (tc::elect_one()) {
        // O2 = Vn_hi Phi^T + Vn_lo Phi^T + Vn_hi Plo^T
        issue_ts(tm + TM_O2, tm + TM_VNHI, sb + ST_PHI, 32, 0, 16, id_n64, 4, false);
        issue_ts(tm + TM_O2, tm + TM_VNLO, sb + ST_PHI, 32, 0, 16, id_n64, 4, true);
        issue_ts(tm + TM_O2, tm + TM_VNHI, sb + ST_PLO, 32, 0, 16, id_n64, 4, true);
        tc::mma_commit(o_full);
        tc::mma_commit(&p_empty[s]);
      }
      __syncwarp();
    }
  }
  } else if (warp < 4 + 4 * NG) {
    tc::reg_set<REGS_CHAIN, REGS_LAUNCH>();
    // ------------------------------------------------------------------ chain epilogue: Vn/Vd conversion and state update
    const int grp = (warp - 4) >> 2;    // column group
    const int quarter = warp & 3;       // TMEM lane quarter this warp may touch
    const int d = quarter * 32 + lane;  // row of H (d_v index)
    const uint32_t lane_addr = tm + ((uint32_t)(quarter * 32) << 16);
    const int64_t tile = ((int64_t)slot * a.Hv + h) * (int64_t)(D * D);
    bool alive = true;

    float2 Hreg[HC / 2];  // H[d][HC*grp + 2w .. +1] = M[HC*grp + 2w .. +1][d]
    // first launch of a chain: part 0 starts from the caller's state, a later part's local chain from zero and its
    // transition chain from the identity
    const float* state_in = !seg_first ? carry + carry_tile : (part == 0 && a.initial_state ? a.initial_state + tile : nullptr);
    float* state_out = seg_last ? (a.final_state ? a.final_state + tile : nullptr) : carry + carry_tile;
    if (phi && seg_first) {
#pragma unroll
      for (int w = 0; w < HC / 2; ++w)
        Hreg[w] = make_float2(HC * grp + 2 * w == d ? 1.f : 0.f, HC * grp + 2 * w + 1 == d ? 1.f : 0.f);
    } else if (state_in != nullptr) {
#pragma unroll
      for (int w = 0; w < HC / 2; ++w)
        Hreg[w] = make_float2(state_in[(int64_t)(HC * grp + 2 * w) * D + d], state_in[(int64_t)(HC * grp + 2 * w + 1) * D + d]);
    } else {
#pragma unroll
      for (int w = 0; w < HC / 2; ++w) Hreg[w] = make_float2(0.f, 0.f);
    }
    auto publish_h = [&]() {
#pragma unroll
      for (int part16 = 0; part16 < HC / 32; ++part16) {  // 16 packed words (32 columns of H) at a time
        uint32_t hi[16], lo[16];
#pragma unroll
        for (int w = 0; w < 16; ++w) split_pair(Hreg[16 * part16 + w], hi[w], lo[w]);
        tc::tmem_st16(lane_addr + TM_HHI + (HC / 2) * grp + 16 * part16, hi);
        tc::tmem_st16(lane_addr + TM_HLO + (HC / 2) * grp + 16 * part16, lo);
      }
      tc::tmem_st_wait();
      tc::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(h_ready);
    };
    publish_h();

    for (int c = 0; c < n_chunks && alive; ++c) {
      const int s = c & 1;
      const uint32_t cp = (uint32_t)c & 1u, u = (uint32_t)(c >> 1);
      const float* scal = reinterpret_cast<const float*>(smem + OFF_SCAL + (c & 3) * SCAL_BYTES);
      if (!tc::mbar_wait_warp(&pfull[s], u & 1u, abort_flag)) { alive = false; break; }  // the scale vectors
      if (!tc::mbar_wait_warp(vn_full, cp, abort_flag)) { alive = false; break; }
      tc::tc_fence_after_sync();
      {
        uint32_t acc[VC];
        tc::tmem_ld_n<VC>(lane_addr + TM_VN + VC * grp, acc);
        float2 v[VC / 2];
        tc::tmem_ld_wait();
#pragma unroll
        for (int w = 0; w < VC / 2; ++w) v[w] = make_float2(__uint_as_float(acc[2 * w]), __uint_as_float(acc[2 * w + 1]));
        {  // Vd first: its columns alias nothing, and the state update waits only for it
          uint32_t dh[VC / 2], dl[VC / 2];
#pragma unroll
          for (int w = 0; w < VC / 2; ++w) {
            const float2 ks = *reinterpret_cast<const float2*>(scal + C + VC * grp + 2 * w);
            split_pair(__fmul2_rn(v[w], ks), dh[w], dl[w]);
          }
          tc::tmem_st_n<VC / 2>(lane_addr + TM_VN + VC * grp, dh);  // into this warp's own accumulator columns
          tc::tmem_st_n<VC / 2>(lane_addr + TM_VN + VC * grp + VC / 2, dl);
          tc::tmem_st_wait();
          tc::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(vd_ready);
        }
        // the Vn images have columns of their own, free once O2 of the previous chunk is complete (long ago)
        if (!tc::mbar_wait_warp(o_full, cp ^ 1u, abort_flag)) { alive = false; break; }
        {
          uint32_t vh[VC / 2], vl[VC / 2];
#pragma unroll
          for (int w = 0; w < VC / 2; ++w) split_pair(v[w], vh[w], vl[w]);
          tc::tmem_st_n<VC / 2>(lane_addr + TM_VNHI + (VC / 2) * grp, vh);
          tc::tmem_st_n<VC / 2>(lane_addr + TM_VNLO + (VC / 2) * grp, vl);
          tc::tmem_st_wait();
          tc::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(vn_ready);
        }
      }
      if (!tc::mbar_wait2(dh_full, cp, o1_done, cp, abort_flag)) { alive = false; break; }
      tc::tc_fence_after_sync();
      {
        const float decay = scal[2 * C];
#pragma unroll
        for (int part32 = 0; part32 < HC / 32; ++part32) {
          uint32_t dh[32];
          tc::tmem_ld32(lane_addr + TM_DH + HC * grp + 32 * part32, dh);
          tc::tmem_ld_wait();
#pragma unroll
          for (int w = 0; w < 16; ++w)
            Hreg[16 * part32 + w] = __ffma2_rn(make_float2(decay, decay), Hreg[16 * part32 + w],
                                               make_float2(__uint_as_float(dh[2 * w]), __uint_as_float(dh[2 * w + 1])));
        }
        publish_h();
      }
    }
    if (alive && state_out != nullptr) {
#pragma unroll
      for (int w = 0; w < HC / 2; ++w) {
        state_out[(int64_t)(HC * grp + 2 * w) * D + d] = Hreg[w].x;
        state_out[(int64_t)(HC * grp + 2 * w + 1) * D + d] = Hreg[w].y;
      }
    }
    if (alive && multi && chain == 0 && c_hi == part_end) {
      // the state that enters part 1, as the fix-up's B operand image (row = d_v, K = d_k): this thread's row, HC / 8 pieces
      uint8_t* img = m0_pack + (((int64_t)n * (plan.parts - 1)) * a.Hv + h) * (int64_t)PACK_BYTES;
#pragma unroll
      for (int j = 0; j < HC / 8; ++j) {
        uint32_t hi[4], lo[4];
#pragma unroll
        for (int w = 0; w < 4; ++w) split_pair(Hreg[4 * j + w], hi[w], lo[w]);
        const uint32_t off = kmajor_piece_off(d, (HC / 8) * grp + j);
        *reinterpret_cast<uint4*>(img + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        *reinterpret_cast<uint4*>(img + D * D * 2 + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
      }
    }
  } else {
    tc::reg_set<REGS_OUT, REGS_LAUNCH>();
    // ------------------------------------------------------------------ output warps: o = scale (qs_i O1 + O2), straight
    // from registers: thread = d_v row, one store per token (a warp covers 32 adjacent features of one token).  When a
    // gated norm follows, the un-normalised output is kept in fp32 scratch for the norm kernel; otherwise it is the result.
    const int quarter = warp & 3;
    const int d = quarter * 32 + lane;
    const uint32_t lane_addr = tm + ((uint32_t)(quarter * 32) << 16);
    float* of = out_f32 ? out_f32 + ((int64_t)sp.b * a.T * a.Hv + h) * D + d : nullptr;
    bool alive = true;
    for (int c = 0; c < n_chunks && alive; ++c) {
      const uint32_t cp = (uint32_t)c & 1u;
      const float* scal = reinterpret_cast<const float*>(smem + OFF_SCAL + (c & 3) * SCAL_BYTES);
      const int len = min(C, sp.len - c * C);
      const int64_t tok0 = sp.t0 + c * C;
      // o_full is committed by the MMA warp after it saw this chunk's stage (tiles and scale vectors) land, so it also
      // orders the scale vectors; waiting on the stage barrier here would alias phases once this warp lags a chunk
      if (!tc::mbar_wait_warp(o_full, cp, abort_flag)) { alive = false; break; }
      tc::tc_fence_after_sync();
      float* pf = of ? of + tok0 * ((int64_t)a.Hv * D) : nullptr;
      __nv_bfloat16* pb = og + tok0 * a.o_stride_t + d;
      const int64_t fstep = (int64_t)a.Hv * D, bstep = a.o_stride_t;
      // O1 is taken whole and released at once: O1 of the next chunk is the first thing the tensor pipe runs while the
      // chain epilogue converts Vn, and must not wait for the stores below.
      uint32_t o1[C];
      tc::tmem_ld32(lane_addr + TM_O1, reinterpret_cast<uint32_t(&)[32]>(o1[0]));
      tc::tmem_ld32(lane_addr + TM_O1 + 32, reinterpret_cast<uint32_t(&)[32]>(o1[32]));
      tc::tmem_ld_wait();
      tc::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(o1_empty);
      // O2 follows in pieces and is folded into the registers that hold O1 (o = qs O1 + O2), so both accumulators are
      // free before the first store: how fast the stores drain no longer decides when the next chunk's output MMAs may run.
      constexpr int PW = 16;  // tokens per piece
#pragma unroll
      for (int piece = 0; piece < C / PW; ++piece) {
        uint32_t o2[PW];
        tc::tmem_ld16(lane_addr + TM_O2 + PW * piece, o2);
        tc::tmem_ld_wait();
        if (piece == C / PW - 1) {  // the accumulator is in registers: the next chunk's MMAs may overwrite it
          tc::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) tc::mbar_arrive(o2_empty);
        }
#pragma unroll
        for (int j4 = 0; j4 < PW / 4; ++j4) {
          const int j = PW * piece + 4 * j4;
          const float4 qs = *reinterpret_cast<const float4*>(scal + j);
          const float2 r0 = __ffma2_rn(make_float2(qs.x, qs.y), make_float2(__uint_as_float(o1[j]), __uint_as_float(o1[j + 1])),
                                       make_float2(__uint_as_float(o2[4 * j4]), __uint_as_float(o2[4 * j4 + 1])));
          const float2 r1 = __ffma2_rn(make_float2(qs.z, qs.w), make_float2(__uint_as_float(o1[j + 2]), __uint_as_float(o1[j + 3])),
                                       make_float2(__uint_as_float(o2[4 * j4 + 2]), __uint_as_float(o2[4 * j4 + 3])));
          o1[j] = __float_as_uint(r0.x); o1[j + 1] = __float_as_uint(r0.y); o1[j + 2] = __float_as_uint(r1.x); o1[j + 3] = __float_as_uint(r1.y);
        }
      }
#pragma unroll
      for (int piece = 0; piece < C / PW; ++piece) {
        float ov[PW];
#pragma unroll
        for (int j = 0; j < PW; ++j) ov[j] = __uint_as_float(o1[PW * piece + j]);
        const int n_here = min(PW, len - PW * piece);  // tokens of this piece that exist
        if (phi) {
          // qt^T of this chunk as bf16 hi and lo images [128 d_k rows][64 tokens] with the 128-byte swizzle: the fix-up
          // reads them, unchanged, as the MN-major A operand of its MMA.  This thread owns row d: two 16-byte pieces.
          uint8_t* img = qt_img + ((int64_t)(c_first + c) * a.Hv + h) * (int64_t)QT_BYTES + d * 128;
#pragma unroll
          for (int e8 = 0; e8 < PW / 8; ++e8) {
            uint32_t hi[4], lo[4];
#pragma unroll
            for (int w = 0; w < 4; ++w) split_pair(make_float2(ov[8 * e8 + 2 * w], ov[8 * e8 + 2 * w + 1]), hi[w], lo[w]);
            const uint32_t off = (uint32_t)((((PW / 8) * piece + e8) ^ (d & 7)) << 4);
            *reinterpret_cast<uint4*>(img + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
            *reinterpret_cast<uint4*>(img + C * D * 2 + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
          }
        } else if (pf != nullptr) {
          if (n_here == PW) {
#pragma unroll
            for (int j = 0; j < PW; ++j) { *pf = ov[j]; pf += fstep; }
          } else {
#pragma unroll
            for (int j = 0; j < PW; ++j) { if (j < n_here) *pf = ov[j]; pf += fstep; }
          }
        } else {
          if (n_here == PW) {
#pragma unroll
            for (int j = 0; j < PW; ++j) { *pb = __float2bfloat16(ov[j]); pb += bstep; }
          } else {
#pragma unroll
            for (int j = 0; j < PW; ++j) { if (j < n_here) *pb = __float2bfloat16(ov[j]); pb += bstep; }
          }
        }
      }
    }
  }

  tc::tc_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag != 0 && a.status != nullptr) atomicOr(a.status, AVE_GDN_DEV_WAIT_EXPIRED);
  if (warp == 1) {
    tc::tc_fence_after_sync();
    tc::tmem_dealloc(tm, 512);
  }
}

// ------------------------------------------------------------------------------------------------ parts: combine and fix-up
// Once every chain of a multi-part sequence has run, the carry buffer holds, per (sequence, value head): chain 0 = the
// true state after part 0, chain 2p-1 = the end state Psi_p of part p's local chain, chain 2p = part p's transition
// matrix F_p (row-major [k][d]: M_end = F_p M0 + Psi_p).
// Serial combine over the parts of one (sequence, value head, 8-column slice of d_v): M0(1) = state after part 0,
// M0(p+1) = F_p M0(p) + Psi_p in fp32 on the CUDA cores; the last one is the sequence's final state.  M0(p) for p >= 2
// also leaves as the bf16 hi/lo operand image the fix-up kernel's MMAs read (B[d_v][k]); the image of M0(1) was written
// by the scan itself.  The steps are serial, so each is kept short: F_p is staged in shared memory with coalesced loads
// (row pitch 129: a thread walks its own row without bank conflicts) and the tile of the next step is already in
// registers while the current one is multiplied.
constexpr int COMBINE_COLS = 8, COMBINE_PITCH = 129;
constexpr size_t COMBINE_SMEM = (size_t)D * COMBINE_PITCH * 4;
__global__ void __launch_bounds__(256)
part_combine_kernel(const AveGdnArgs a, const int32_t* __restrict__ chunk_start, const float* __restrict__ carry,
                    uint8_t* __restrict__ m0_pack, const __grid_constant__ ScanPlan plan) {
  extern __shared__ float Fs[];  // [D][COMBINE_PITCH]
  __shared__ __align__(16) float cur[2][D][COMBINE_COLS];
  const int cb = blockIdx.x, h = blockIdx.y, n = blockIdx.z, tid = threadIdx.x;
  if (a.cu_seqlens != nullptr && chunk_start[a.n_seqs] < 0) return;
  const SeqSpan sp = seq_span(a.cu_seqlens, n, a.T, nullptr);
  if (!sp.ok || (a.cu_seqlens != nullptr && a.max_seqlen > 0 && sp.len > a.max_seqlen)) return;
  const int seq_chunks = (sp.len + C - 1) / C;
  if (seq_chunks <= plan.part_begin[1]) return;  // a plain chain: the scan wrote the final state itself
  const int slot = a.state_indices ? a.state_indices[n] : n;
  if (slot < 0 || slot >= a.num_slots) return;
  int active = 1;
  for (int p = 1; p < plan.parts; ++p) active += plan.part_begin[p] < seq_chunks ? 1 : 0;
  if (active == 2 && a.final_state == nullptr) return;  // nothing to produce
  const int chains = 2 * plan.parts - 1;
  auto tile_of = [&](int chain) { return carry + (((int64_t)n * chains + chain) * a.Hv + h) * (int64_t)(D * D); };
  {
    const float* src = tile_of(0);
    for (int e = tid; e < D * COMBINE_COLS; e += 256) cur[0][e / COMBINE_COLS][e % COMBINE_COLS] = src[(e / COMBINE_COLS) * D + cb * COMBINE_COLS + e % COMBINE_COLS];
  }
  // a thread fetches 16 float4 of the 128x128 tile: element 4 * (tid + 256 i), i.e. row (tid + 256 i) / 32
  float4 pre[16], psi_pre;
  auto fetch = [&](int p) {
    const float4* F4 = reinterpret_cast<const float4*>(tile_of(2 * p));
#pragma unroll
    for (int i = 0; i < 16; ++i) pre[i] = F4[tid + 256 * i];
    psi_pre = *reinterpret_cast<const float4*>(tile_of(2 * p - 1) + (int64_t)(tid >> 1) * D + cb * COMBINE_COLS + (tid & 1) * 4);
  };
  fetch(1);
  int b = 0;
  for (int p = 1; p < active; ++p) {
    __syncthreads();  // the previous step's readers of Fs are done
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int e = 4 * (tid + 256 * i), row = e >> 7, c0 = e & 127;
      float* dst = Fs + row * COMBINE_PITCH + c0;
      dst[0] = pre[i].x; dst[1] = pre[i].y; dst[2] = pre[i].z; dst[3] = pre[i].w;
    }
    const float4 psi = psi_pre;
    if (p + 1 < active) fetch(p + 1);
    __syncthreads();
    {  // next = F_p cur + Psi_p: a thread owns one row k and four columns
      const int k = tid >> 1, j0 = (tid & 1) * 4;
      const float* Frow = Fs + k * COMBINE_PITCH;
      float acc0 = psi.x, acc1 = psi.y, acc2 = psi.z, acc3 = psi.w;
#pragma unroll 16
      for (int d = 0; d < D; ++d) {
        const float f = Frow[d];
        const float4 c4 = *reinterpret_cast<const float4*>(&cur[b][d][j0]);
        acc0 = fmaf(f, c4.x, acc0); acc1 = fmaf(f, c4.y, acc1); acc2 = fmaf(f, c4.z, acc2); acc3 = fmaf(f, c4.w, acc3);
      }
      *reinterpret_cast<float4*>(&cur[b ^ 1][k][j0]) = make_float4(acc0, acc1, acc2, acc3);
    }
    b ^= 1;
    __syncthreads();
    if (p + 1 < active && tid < 128) {  // operand image of M0(p+1): B[row = d_v][k] = M0[k][d_v]; a 16-byte piece of hi and of lo
      const int k8 = tid >> 3, v = tid & 7;
      uint32_t hi[4], lo[4];
#pragma unroll
      for (int w = 0; w < 4; ++w) split_pair(make_float2(cur[b][8 * k8 + 2 * w][v], cur[b][8 * k8 + 2 * w + 1][v]), hi[w], lo[w]);
      uint8_t* img = m0_pack + (((int64_t)n * (plan.parts - 1) + p) * a.Hv + h) * (int64_t)PACK_BYTES;
      const uint32_t off = kmajor_piece_off(cb * COMBINE_COLS + v, k8);
      *reinterpret_cast<uint4*>(img + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
      *reinterpret_cast<uint4*>(img + D * D * 2 + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    }
  }
  __syncthreads();
  if (a.final_state != nullptr) {
    float* dst = a.final_state + ((int64_t)slot * a.Hv + h) * (int64_t)(D * D);
    for (int e = tid; e < D * COMBINE_COLS; e += 256) dst[(e / COMBINE_COLS) * D + cb * COMBINE_COLS + e % COMBINE_COLS] = cur[b][e / COMBINE_COLS][e % COMBINE_COLS];
  }
}

// Fix-up of the parts after the first.  For 128 tokens (two chunks of one part) of one value head,
//   o = o_local + qt M0(part)        (qt = the transition chain's rows, [128 tokens][128 d_k])
// is one 128x128x128 product on tcgen05 with both operands as bf16 hi+lo pairs (hi hi + hi lo + lo hi): A = the qt^T
// images the scan wrote (MN-major, brought in by bulk copies), B = the image of M0(part).  The accumulator (a thread
// per token row) is staged through shared memory so that everything that touches global memory runs in the layout of
// the streaming norm kernel: a half-warp per token row, 8 adjacent features per lane, 16- and 32-byte accesses, the
// RMS over d_v as four shuffles.  (Reading o_local and z straight from the accumulator's layout, a row or a column per
// thread, measured three to four times slower: 2- or 4-byte accesses and tens of instructions per element.)
// A CTA serves one (sequence, part, head) and walks every `gridDim.x`-th pair of chunks with the M0 image resident; the
// images of the next pair are in flight while the current pair's rows are streamed.
constexpr int FIN_THREADS = 512;
constexpr int FIN_PITCH = 132;  // floats per staged row: 16-byte aligned rows that spread over the banks
constexpr int FIN_A = 0, FIN_B = 65536, FIN_STAGE = FIN_B + PACK_BYTES, FIN_BARS = FIN_STAGE + 128 * FIN_PITCH * 4;
constexpr size_t FIN_SMEM = FIN_BARS + 64 + 1024;
__global__ void __launch_bounds__(FIN_THREADS, 1)
part_finish_kernel(const AveGdnArgs a, const int32_t* __restrict__ chunk_start, const float* __restrict__ o_f32,
                   const uint8_t* __restrict__ qt_img, const uint8_t* __restrict__ m0_pack, const __grid_constant__ ScanPlan plan) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  float* stage = reinterpret_cast<float*>(smem + FIN_STAGE);  // [128 tokens][FIN_PITCH] product rows
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + FIN_BARS);
  uint64_t* b_bar = bars;
  uint64_t* a_full = bars + 1;
  uint64_t* mma_bar = bars + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  const int h = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n = blockIdx.z / (plan.parts - 1), part = 1 + blockIdx.z % (plan.parts - 1);
  if (a.cu_seqlens != nullptr && chunk_start[a.n_seqs] < 0) return;
  const SeqSpan sp = seq_span(a.cu_seqlens, n, a.T, nullptr);
  if (!sp.ok || (a.cu_seqlens != nullptr && a.max_seqlen > 0 && sp.len > a.max_seqlen)) return;
  const int seq_chunks = (sp.len + C - 1) / C;
  const int c_begin = plan.part_begin[part], c_end = min(plan.part_begin[part + 1], seq_chunks);
  const int n_pairs = (c_end - c_begin + 1) / 2;  // part boundaries are even, so a pair never straddles two parts
  if ((int)blockIdx.x >= n_pairs) return;
  const int slot = a.state_indices ? a.state_indices[n] : n;
  const bool skipped = slot < 0 || slot >= a.num_slots;  // the scan skipped the sequence: its rows are zero
  const int64_t rec0 = a.cu_seqlens ? chunk_start[n] : (int64_t)n * ((a.T + C - 1) / C);  // record of the sequence's chunk 0
  const int stride = gridDim.x;

  auto load_qt = [&](int pair) {  // called by one thread
    const int c0 = c_begin + 2 * pair, cnt = min(2, c_end - c0);
    tc::mbar_expect_tx(a_full, (uint32_t)(cnt * QT_BYTES));
    for (int i = 0; i < cnt; ++i) {
      const uint8_t* img = qt_img + ((rec0 + c0 + i) * a.Hv + h) * (int64_t)QT_BYTES;
      tc::bulk_load(smem + FIN_A + i * 16384, img, 16384, a_full);                   // hi: [chunk 0 | chunk 1]
      tc::bulk_load(smem + FIN_A + 32768 + i * 16384, img + 16384, 16384, a_full);   // lo: [chunk 0 | chunk 1]
    }
  };
  if (tid == 0) {
    tc::mbar_init(b_bar, 1);
    tc::mbar_init(a_full, 1);
    tc::mbar_init(mma_bar, 1);
    *abort_flag = 0;
    tc::fence_barrier_init();
    if (!skipped) {
      const uint8_t* img = m0_pack + (((int64_t)n * (plan.parts - 1) + (part - 1)) * a.Hv + h) * (int64_t)PACK_BYTES;
      tc::mbar_expect_tx(b_bar, PACK_BYTES);
      tc::bulk_load(smem + FIN_B, img, PACK_BYTES, b_bar);
      load_qt(blockIdx.x);
    }
  }
  if (warp == 1) tc::tmem_alloc(tmem_slot, 128);
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tm = *tmem_slot;
  const int quarter = warp & 3, colq = warp >> 2;  // accumulator: TMEM lane quarter (token rows) and column quarter of this warp
  const int hw = tid >> 4, sub = tid & 15;          // streaming pass: half-warp index (32 of them) and lane inside it
  const bool gate_first = (a.flags & AVE_GDN_FLAG_GATE_FIRST) != 0;
  float2 wv[4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    wv[i] = a.norm_weight ? make_float2(a.norm_weight[8 * sub + 2 * i], a.norm_weight[8 * sub + 2 * i + 1]) : make_float2(1.f, 1.f);
  bool ok = true;

  int it = 0;
  for (int pair = blockIdx.x; pair < n_pairs && ok; pair += stride, ++it) {
    const int c0 = c_begin + 2 * pair;
    const int64_t tok0 = sp.t0 + (int64_t)c0 * C;
    const int rows = min(min(2, c_end - c0) * C, sp.len - c0 * C);
    if (!skipped) {
      if (warp == 0) {
        bool landed = it > 0 || tc::mbar_wait_warp(b_bar, 0, abort_flag);
        landed = landed && tc::mbar_wait_warp(a_full, (uint32_t)it & 1u, abort_flag);
        tc::tc_fence_after_sync();
        if (landed && tc::elect_one()) {
          constexpr uint32_t idesc = tc::idesc_f16(128, 128, 1, 1, true, false);  // A MN-major (token rows), B K-major
          const uint32_t sa = tc::smem_u32(smem + FIN_A), sb = tc::smem_u32(smem + FIN_B);
#pragma unroll
          for (int t = 0; t < 3; ++t) {  // hi hi, hi lo, lo hi
            const uint32_t ab = sa + (t == 2 ? 32768u : 0u), bb = sb + (t == 1 ? 32768u : 0u);
#pragma unroll
            for (int k = 0; k < 8; ++k)  // 16 d_k rows of qt^T per step: 2048 bytes; the two chunks' images lie 16384 bytes apart
              tc::mma_ss(tm, tc::smem_desc_sw128(ab + k * 2048, 16384, 1024),
                         tc::smem_desc_sw128(bb + (uint32_t)((k >> 2) * 16384 + (k & 3) * 32), 16, 1024), idesc, (t | k) != 0 ? 1u : 0u);
          }
          tc::mma_commit(mma_bar);
        }
        __syncwarp();
      }
      ok = tc::mbar_wait(mma_bar, (uint32_t)it & 1u, abort_flag);
      tc::tc_fence_after_sync();
      // the images have been read: the next pair's take their place while this pair is finished
      if (ok && tid == 0 && pair + stride < n_pairs) load_qt(pair + stride);
      if (ok) {  // accumulator row -> staged row (this warp: 32 token rows x 32 columns)
        uint32_t acc[32];
        tc::tmem_ld32(tm + ((uint32_t)(quarter * 32) << 16) + 32 * colq, acc);
        tc::tmem_ld_wait();
        float* dstrow = stage + (quarter * 32 + lane) * FIN_PITCH + 32 * colq;
#pragma unroll
        for (int i = 0; i < 8; ++i)
          *reinterpret_cast<uint4*>(dstrow + 4 * i) = make_uint4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
      }
    }
    tc::tc_fence_before_sync();
    ok = __syncthreads_and(ok ? 1 : 0) != 0;  // staged rows complete; the accumulator is free for the next product
    tc::tc_fence_after_sync();
    if (ok) {
      // streaming pass: this half-warp takes token rows hw, hw + 32, hw + 64, hw + 96
      float2 x[4][4];
      uint4 zraw[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int r = hw + 32 * u;
        const bool live = r < rows;
        if (!skipped && live) {
          const float* ol = o_f32 + (((int64_t)sp.b * a.T + tok0 + r) * a.Hv + h) * D + 8 * sub;
          const float4 o0 = *reinterpret_cast<const float4*>(ol), o1 = *reinterpret_cast<const float4*>(ol + 4);
          const float4 p0 = *reinterpret_cast<const float4*>(stage + r * FIN_PITCH + 8 * sub);
          const float4 p1 = *reinterpret_cast<const float4*>(stage + r * FIN_PITCH + 8 * sub + 4);
          x[u][0] = make_float2(o0.x + p0.x, o0.y + p0.y); x[u][1] = make_float2(o0.z + p0.z, o0.w + p0.w);
          x[u][2] = make_float2(o1.x + p1.x, o1.y + p1.y); x[u][3] = make_float2(o1.z + p1.z, o1.w + p1.w);
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) x[u][i] = make_float2(0.f, 0.f);
        }
        zraw[u] = make_uint4(0u, 0u, 0u, 0u);
        if (a.z != nullptr && live)
          zraw[u] = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(a.z) + sp.b * a.z_stride_b +
                                                    (tok0 + r) * a.z_stride_t + (int64_t)h * a.z_stride_h + 8 * sub);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int r = hw + 32 * u;
        uint32_t packed[4];
        if (a.z != nullptr) {
          float2 gate[4] = {silu2(bf16x2_to_float2(zraw[u].x)), silu2(bf16x2_to_float2(zraw[u].y)),
                            silu2(bf16x2_to_float2(zraw[u].z)), silu2(bf16x2_to_float2(zraw[u].w))};
          float2 ss2 = make_float2(0.f, 0.f);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            if (gate_first) x[u][i] = __fmul2_rn(x[u][i], gate[i]);
            ss2 = __ffma2_rn(x[u][i], x[u][i], ss2);
          }
          float ss = ss2.x + ss2.y;
#pragma unroll
          for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);  // stays inside the half-warp
          const float rinv = rsqrtf(ss * (1.0f / D) + a.norm_eps);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float2 y2 = __fmul2_rn(__fmul2_rn(x[u][i], make_float2(rinv, rinv)), wv[i]);
            if (!gate_first) y2 = __fmul2_rn(y2, gate[i]);
            packed[i] = pack_bf16x2(y2.x, y2.y);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) packed[i] = pack_bf16x2(x[u][i].x, x[u][i].y);
        }
        if (r < rows)
          *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.o) + sp.b * a.o_stride_b + (tok0 + r) * a.o_stride_t +
                                    (int64_t)h * a.o_stride_h + 8 * sub) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      }
    }
    __syncthreads();  // the staged rows have been read: the next pair may overwrite them
  }
  tc::tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0u && tid == 0 && a.status != nullptr) atomicOr(a.status, AVE_GDN_DEV_WAIT_EXPIRED);
  if (warp == 1) {
    tc::tc_fence_after_sync();
    tc::tmem_dealloc(tm, 128);
  }
}

// ------------------------------------------------------------------------------------------------ schedule and scratch
constexpr int SEG_FIRST_DIV = 16;   // first range = 1/16 of the longest chain's chunks
constexpr int SEG_GROWTH_X4 = 12;   // each range 3x the one before (in quarters)
constexpr int SEG_MAX = 8;
constexpr int PART0_X4 = 4;         // length of part 0 in quarters of a later part's length
constexpr int NUM_SMS = 148;        // B200; the schedule is a pure function of the arguments, so that the workspace
                                    // query and the launch agree without a device being current
struct WsLayout {
  size_t chunk_start, w_hi, w_lo, p_hi, p_lo, tu_hi, tu_lo, scal, o_f32, qt_img, carry, m0_pack, total;
  int64_t chunks;
  int max_chunks;      // bound of the longest sequence, in chunks
  int parts;           // see ScanPlan
  int part_begin[MAX_PARTS + 1];
  int segments;        // chunk ranges handled by separate launches
  int seg_begin[9];    // range i covers chunk offsets [seg_begin[i], seg_begin[i+1]) inside every part
};

// `plain`: one part, one range, everything on the caller's stream (the schedule of the fixed-scratch entry point).
WsLayout ws_layout(const AveGdnArgs& a, bool plain) {
  WsLayout L;
  L.chunks = a.cu_seqlens ? (int64_t)a.T / C + a.n_seqs : (int64_t)a.B * ((a.T + C - 1) / C);
  const size_t recs = (size_t)L.chunks * a.Hv;
  auto up = [](size_t x) { return (x + 1023) & ~(size_t)1023; };
  size_t off = 0;
  L.chunk_start = off; off = up(off + (2 * (size_t)a.n_seqs + 1 + (size_t)L.chunks) * 4);  // prefix table, chunk -> sequence map, scan order
  L.w_hi = off; off = up(off + recs * REC_W);
  L.w_lo = off; off = up(off + recs * REC_W);
  L.p_hi = off; off = up(off + recs * REC_P);
  L.p_lo = off; off = up(off + recs * REC_P);
  L.tu_hi = off; off = up(off + recs * REC_P);
  L.tu_lo = off; off = up(off + recs * REC_P);
  L.scal = off; off = up(off + recs * (size_t)(SCAL_FLOATS * 4));
  // The longest chain is known for dense batches and for packed ones that come with the max_seqlen bound; otherwise only
  // its bound T is.
  const int max_chunks = ((a.cu_seqlens != nullptr && a.max_seqlen > 0 ? min(a.max_seqlen, a.T) : a.T) + C - 1) / C;
  L.max_chunks = max_chunks;
  const int64_t heads_total = (int64_t)a.n_seqs * a.Hv;
  const bool push = a.o_peers != nullptr && a.n_peers > 1;
  // Parts: with few long chains most SMs idle while every chain walks its chunks one after the other.  Cutting the
  // sequences into S parts that run at the same time shortens the walk S-fold at the price of a second (transition)
  // chain per later part and one GEMM-shaped fix-up; S is the largest count whose 2S-1 chains per head still get an SM
  // each.  Not with the fused all-gather: there the fix-up would push most rows to the peers after the scan instead of
  // beside it.
  L.parts = 1;
  if (!plain && !push && max_chunks >= 32) {
    const int64_t per_head = (NUM_SMS / (heads_total > 0 ? heads_total : 1) + 1) / 2;  // chains per head that still get an SM each: 2S - 1
    int S = per_head < MAX_PARTS ? (int)per_head : MAX_PARTS;
    while (S > 1 && max_chunks / S < 16) --S;
    // Two parts only halve the walk and pay for it with a third as many chains again plus the fix-up of half the rows:
    // measured break-even (32 heads, 8192 tokens: 0.46 ms either way).  From three parts on the cut wins: 4 / 8 / 16 heads
    // at 32768 tokens run 3.0x / 2.0x / 1.3x faster than the plain chain.
    L.parts = S >= 3 ? S : 1;
  }
  L.part_begin[0] = 0;
  {
    // Part 0 runs one chain and needs no fix-up, a later part runs two chains and its rows wait for the fix-up, so
    // part 0 is made PART0_X4 / 4 times as long as the others; lengths are even (the fix-up works on pairs of chunks).
    const int len = max(2, (4 * max_chunks / (4 * (L.parts - 1) + PART0_X4) + 1) & ~1);
    const int first = L.parts > 1 ? max(2, (max_chunks - (L.parts - 1) * len + 1) & ~1) : 0;
    for (int p = 1; p <= MAX_PARTS; ++p) L.part_begin[p] = p < L.parts ? first + (p - 1) * len : (1 << 24);
  }
  int part_len = 0;  // the longest part, in chunks
  for (int p = 0; p < L.parts; ++p) part_len = max(part_len, min(L.part_begin[p + 1], max_chunks) - L.part_begin[p]);
  L.o_f32 = off;
  if (a.z != nullptr || L.parts > 1) off = up(off + (size_t)a.B * a.T * a.Hv * D * 4);  // rows waiting for the norm / the fix-up
  L.qt_img = off;
  if (L.parts > 1) off = up(off + recs * (size_t)QT_BYTES);                             // the transition chains' rows (operand images)
  // Ranges: few long chains (fewer scan CTAs than half the SMs, or parts): pass 1 of range i+1 runs on the idle SMs
  // while pass 2 of range i walks its chains.  The state crosses ranges through the carry buffer.  (Also switching them
  // on for packed batches whose longest chain exceeds 1.5 times an SM's share of all chunk-heads was measured on an
  // eighth of the heads of the 256K-token batch, 256 chains: 1.38 ms against 1.15 ms without ranges.)
  const bool chain_bound = heads_total <= 74;
  L.seg_begin[0] = 0;
  if (plain || !(chain_bound && max_chunks >= 32)) {
    L.segments = 1;
    L.seg_begin[1] = 1 << 24;  // every chunk (times 64 still fits an int)
  } else {
    // A short first range (its pass 1 is the only one nothing overlaps), then ranges that grow geometrically: pass 1
    // of a range must fit inside pass 2 of the range before it.
    // With the fused all-gather the gated norm of a range also pushes that range's rows to every peer over NVLink,
    // which takes about as long as the chain itself; only the last range's push is exposed, so the ranges are equal
    // and as many as the event pool allows instead of growing.
    int len = push ? (part_len + SEG_MAX - 1) / SEG_MAX : max(1, (part_len + SEG_FIRST_DIV - 1) / SEG_FIRST_DIV);
    L.segments = 0;
    while (L.seg_begin[L.segments] < part_len) {
      int next = L.seg_begin[L.segments] + len;
      if (L.segments == SEG_MAX - 1 || next >= part_len) next = part_len;
      L.seg_begin[++L.segments] = next;
      if (!push) len = max(len + 1, len * SEG_GROWTH_X4 / 4);
    }
  }
  L.carry = off;
  if (L.segments > 1 || L.parts > 1) off = up(off + (size_t)a.n_seqs * (2 * L.parts - 1) * a.Hv * D * D * 4);
  L.m0_pack = off;
  if (L.parts > 1) off = up(off + (size_t)a.n_seqs * (L.parts - 1) * a.Hv * PACK_BYTES);
  L.total = off;
  return L;
}

}  // namespace

int launch_gated_rmsnorm_f32in_batched(const AveGdnNormArgs& a, cudaStream_t stream, const void* const* peers, int n_peers,
                                       int64_t peer_off, int batches, int64_t xs_b, int64_t zs_b, int64_t ys_b);

size_t prefill_tc_workspace_bytes(const AveGdnArgs& a, bool plain) { return ws_layout(a, plain).total; }

// Kernels one call enqueues, mirroring launch_prefill_tc below.
int prefill_tc_launch_count(const AveGdnArgs& a, bool plain) {
  const WsLayout L = ws_layout(a, plain);
  if (L.chunks == 0 || a.n_seqs == 0) return 0;
  const bool push = a.o_peers != nullptr && a.n_peers > 1;
  const int norm_launch = (push || a.B == 1) ? 1 : a.B;  // norm_rows: one launch, or one per batch row
  int n = a.cu_seqlens != nullptr ? 1 : 0;                 // chunk table
  n += 2 * L.segments;                                     // pass 1 and pass 2 of every range
  if (a.z != nullptr) n += (a.cu_seqlens == nullptr ? L.segments : 1) * norm_launch;
  if (L.parts > 1) n += 2;                                 // combine and fix-up
  return n;
}

// Helper streams and events for the range-overlapped schedule.  Pass 2 runs on a high-priority stream so that, when a
// range's pass 1 completes and both its pass 2 and the next range's pass 1 become runnable, the few whole-SM pass-2
// CTAs are placed first.  Each device owns a small pool of such sets; a call takes the set its stream hashes to, so
// calls on different streams usually overlap instead of queueing behind one another's helper streams.  A device's sets
// and the whole enqueue sequence of a call are guarded by that device's mutex: the record/wait pairs of two host
// threads never interleave, which is what makes a set shareable at all (a wait binds to the event's latest record at
// the time of the call).
struct SideSet {
  cudaStream_t prep = nullptr, scan = nullptr, norm = nullptr;
  cudaEvent_t fork = nullptr, join = nullptr, join_norm = nullptr, chains_done = nullptr, combined = nullptr;
  cudaEvent_t done[SEG_MAX] = {}, scanned[SEG_MAX] = {};
  bool ready = false;
};
constexpr int SIDE_SETS = 4, MAX_DEVICES = 64;
struct DeviceSide {
  std::mutex mu;
  SideSet sets[SIDE_SETS];
  bool attr_set = false;
};
static DeviceSide g_side[MAX_DEVICES];

static void destroy_side_set(SideSet& s) {
  if (s.prep) cudaStreamDestroy(s.prep);
  if (s.scan) cudaStreamDestroy(s.scan);
  if (s.norm) cudaStreamDestroy(s.norm);
  for (cudaEvent_t e : {s.fork, s.join, s.join_norm, s.chains_done, s.combined}) if (e) cudaEventDestroy(e);
  for (int i = 0; i < SEG_MAX; ++i) { if (s.done[i]) cudaEventDestroy(s.done[i]); if (s.scanned[i]) cudaEventDestroy(s.scanned[i]); }
  s = SideSet{};
}
// Called with the device's mutex held.  A set is built in a local and published only when every piece exists.
static SideSet* side_set(DeviceSide& dev, cudaStream_t stream) {
  SideSet& slot = dev.sets[(reinterpret_cast<uintptr_t>(stream) >> 4) % SIDE_SETS];
  if (slot.ready) return &slot;
  SideSet s;
  int lo = 0, hi = 0;
  bool ok = cudaDeviceGetStreamPriorityRange(&lo, &hi) == cudaSuccess;
  ok = ok && cudaStreamCreateWithPriority(&s.prep, cudaStreamNonBlocking, lo) == cudaSuccess;
  ok = ok && cudaStreamCreateWithPriority(&s.scan, cudaStreamNonBlocking, hi) == cudaSuccess;
  ok = ok && cudaStreamCreateWithPriority(&s.norm, cudaStreamNonBlocking, lo) == cudaSuccess;
  ok = ok && cudaEventCreateWithFlags(&s.fork, cudaEventDisableTiming) == cudaSuccess;
  ok = ok && cudaEventCreateWithFlags(&s.join, cudaEventDisableTiming) == cudaSuccess;
  ok = ok && cudaEventCreateWithFlags(&s.join_norm, cudaEventDisableTiming) == cudaSuccess;
  ok = ok && cudaEventCreateWithFlags(&s.chains_done, cudaEventDisableTiming) == cudaSuccess;
  ok = ok && cudaEventCreateWithFlags(&s.combined, cudaEventDisableTiming) == cudaSuccess;
  for (int i = 0; i < SEG_MAX; ++i) {
    ok = ok && cudaEventCreateWithFlags(&s.done[i], cudaEventDisableTiming) == cudaSuccess;
    ok = ok && cudaEventCreateWithFlags(&s.scanned[i], cudaEventDisableTiming) == cudaSuccess;
  }
  if (!ok) { destroy_side_set(s); return nullptr; }
  s.ready = true;
  slot = s;
  return &slot;
}

// Gated RMSNorm over the fp32 output for tokens [t_begin, t_end) of every batch row, one launch.
static int norm_rows(const AveGdnArgs& a, float* o_f32, int t_begin, int t_end, cudaStream_t stream) {
  if (t_end <= t_begin) return AVE_GDN_OK;
  AveGdnNormArgs nb{};
  nb.struct_size = sizeof(nb);
  nb.flags = a.flags & AVE_GDN_FLAG_GATE_FIRST;
  nb.rows = (int64_t)(t_end - t_begin) * a.Hv;
  nb.d = D; nb.heads = a.Hv; nb.eps = a.norm_eps; nb.weight = a.norm_weight;
  nb.x = o_f32 + (int64_t)t_begin * a.Hv * D;
  nb.x_stride_t = (int64_t)a.Hv * D; nb.x_stride_h = D;
  nb.z = reinterpret_cast<const __nv_bfloat16*>(a.z) + (int64_t)t_begin * a.z_stride_t;
  nb.z_stride_t = a.z_stride_t; nb.z_stride_h = a.z_stride_h;
  nb.y = reinterpret_cast<__nv_bfloat16*>(a.o) + (int64_t)t_begin * a.o_stride_t;
  nb.y_stride_t = a.o_stride_t; nb.y_stride_h = a.o_stride_h;
  // With peers the launch covers every batch row at once (many short launches keep too few peer stores in flight);
  // without, one launch per batch row measured 1-2 % faster on four rows of a million norm rows each.
  const bool push = a.o_peers != nullptr && a.n_peers > 1;
  const int64_t xs_b = (int64_t)a.T * a.Hv * D;
  if (push || a.B == 1)
    return launch_gated_rmsnorm_f32in_batched(nb, stream, a.o_peers, a.n_peers, (int64_t)t_begin * a.o_stride_t, a.B, xs_b,
                                              a.z_stride_b, a.o_stride_b);
  for (int b = 0; b < a.B; ++b) {
    AveGdnNormArgs one = nb;
    one.x = reinterpret_cast<const float*>(nb.x) + b * xs_b;
    one.z = reinterpret_cast<const __nv_bfloat16*>(nb.z) + b * a.z_stride_b;
    one.y = reinterpret_cast<__nv_bfloat16*>(nb.y) + b * a.o_stride_b;
    const int rc = launch_gated_rmsnorm_f32in_batched(one, stream, a.o_peers, a.n_peers,
                                                      (int64_t)b * a.o_stride_b + (int64_t)t_begin * a.o_stride_t, 1, 0, 0, 0);
    if (rc != AVE_GDN_OK) return rc;
  }
  return AVE_GDN_OK;
}

// Enqueues one prefill.  Thread-safe: the enqueue sequence of a call runs under the device's mutex (see SideSet).
int launch_prefill_tc(const AveGdnArgs& a, cudaStream_t stream, bool plain) {
  const WsLayout L = ws_layout(a, plain);
  if (L.chunks == 0 || a.n_seqs == 0) return AVE_GDN_OK;
  char* ws = reinterpret_cast<char*>(a.workspace);
  int32_t* chunk_start = reinterpret_cast<int32_t*>(ws + L.chunk_start);
  PrepOut po;
  po.w_hi = reinterpret_cast<__nv_bfloat16*>(ws + L.w_hi);
  po.w_lo = reinterpret_cast<__nv_bfloat16*>(ws + L.w_lo);
  po.p_hi = reinterpret_cast<__nv_bfloat16*>(ws + L.p_hi);
  po.p_lo = reinterpret_cast<__nv_bfloat16*>(ws + L.p_lo);
  po.tu_hi = reinterpret_cast<__nv_bfloat16*>(ws + L.tu_hi);
  po.tu_lo = reinterpret_cast<__nv_bfloat16*>(ws + L.tu_lo);
  po.scal = reinterpret_cast<float*>(ws + L.scal);

  GdnMaps maps;
  {
    int rc;
    const uint32_t box4[4] = {64, 1, 64, 1};
    const uint64_t dq[4] = {D, (uint64_t)a.Hk, (uint64_t)a.T, (uint64_t)a.B};
    const uint64_t sq[4] = {2, (uint64_t)a.q_stride_h * 2, (uint64_t)a.q_stride_t * 2, (uint64_t)(a.B > 1 ? a.q_stride_b : a.q_stride_t * a.T) * 2};
    const uint64_t sk[4] = {2, (uint64_t)a.k_stride_h * 2, (uint64_t)a.k_stride_t * 2, (uint64_t)(a.B > 1 ? a.k_stride_b : a.k_stride_t * a.T) * 2};
    if ((rc = make_tmap(&maps.q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(a.q), 4, dq, sq, box4, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
    if ((rc = make_tmap(&maps.k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(a.k), 4, dq, sk, box4, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
    const uint32_t boxv[4] = {64, 1, 64, 1};
    const uint64_t dv4[4] = {D, (uint64_t)a.Hv, (uint64_t)a.T, (uint64_t)a.B};
    const uint64_t sv[4] = {2, (uint64_t)a.v_stride_h * 2, (uint64_t)a.v_stride_t * 2, (uint64_t)(a.B > 1 ? a.v_stride_b : a.v_stride_t * a.T) * 2};
    if ((rc = make_tmap(&maps.v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(a.v), 4, dv4, sv, boxv, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  }

  int dev_id = 0;
  AVE_CUDA_TRY(cudaGetDevice(&dev_id));
  if (dev_id < 0 || dev_id >= MAX_DEVICES) return AVE_GDN_UNSUPPORTED;
  DeviceSide& dev = g_side[dev_id];
  std::lock_guard<std::mutex> guard(dev.mu);
  if (!dev.attr_set) {
    AVE_CUDA_TRY(cudaFuncSetAttribute(chunk_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PREP_SMEM));
    AVE_CUDA_TRY(cudaFuncSetAttribute(chunk_scan_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SCAN_SMEM));
    AVE_CUDA_TRY(cudaFuncSetAttribute(chunk_scan_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SCAN_SMEM));
    AVE_CUDA_TRY(cudaFuncSetAttribute(part_finish_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FIN_SMEM));
    AVE_CUDA_TRY(cudaFuncSetAttribute(part_combine_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)COMBINE_SMEM));
    dev.attr_set = true;
  }
  if (a.cu_seqlens != nullptr) {
    chunk_table_tc_kernel<<<1, 1024, 0, stream>>>(a.cu_seqlens, a.n_seqs, a.T, chunk_start, (int)L.chunks, a.status);
    AVE_CUDA_TRY(cudaGetLastError());
  }
  float* o_f32 = (a.z != nullptr || L.parts > 1) ? reinterpret_cast<float*>(ws + L.o_f32) : nullptr;
  uint8_t* qt_img = L.parts > 1 ? reinterpret_cast<uint8_t*>(ws + L.qt_img) : nullptr;
  float* carry = reinterpret_cast<float*>(ws + L.carry);
  uint8_t* m0_pack = reinterpret_cast<uint8_t*>(ws + L.m0_pack);
  const int32_t* seq_order = a.cu_seqlens ? chunk_start + a.n_seqs + 1 + L.chunks : nullptr;
  ScanPlan plan;
  plan.parts = L.parts;
  for (int p = 0; p <= MAX_PARTS; ++p) plan.part_begin[p] = L.part_begin[p];
  const unsigned scan_grid = (unsigned)a.n_seqs * (unsigned)(2 * L.parts - 1) * (unsigned)a.Hv;
  const int part0_tokens = L.parts > 1 ? min(a.T, L.part_begin[1] * C) : a.T;  // tokens no fix-up touches (dense layout)

  // combine + fix-up of the later parts, after every chain has finished (parts > 1 only).  The image of M0(1) comes from
  // the scan, so with two parts the fix-up needs nothing from the combine, which then only produces the final states
  // and runs on `side_stream` (when given) beside the fix-up.
  auto finish_parts = [&](cudaStream_t s, cudaStream_t side_stream, cudaEvent_t scanned, cudaEvent_t combined) -> int {
    if (L.parts <= 1) return AVE_GDN_OK;
    plan.r0 = 0; plan.rn = 1 << 24;
    const dim3 cgrid(D / COMBINE_COLS, (unsigned)a.Hv, (unsigned)a.n_seqs);
    const bool beside = L.parts == 2 && side_stream != nullptr;
    if (beside) {
      AVE_CUDA_TRY(cudaEventRecord(scanned, s));
      AVE_CUDA_TRY(cudaStreamWaitEvent(side_stream, scanned, 0));
      part_combine_kernel<<<cgrid, 256, COMBINE_SMEM, side_stream>>>(a, chunk_start, carry, m0_pack, plan);
      AVE_CUDA_TRY(cudaGetLastError());
      AVE_CUDA_TRY(cudaEventRecord(combined, side_stream));
    } else {
      part_combine_kernel<<<cgrid, 256, COMBINE_SMEM, s>>>(a, chunk_start, carry, m0_pack, plan);
      AVE_CUDA_TRY(cudaGetLastError());
    }
    int part_len = 0;  // the longest of the later parts
    for (int p = 1; p < L.parts; ++p) part_len = max(part_len, min(L.part_begin[p + 1], L.max_chunks) - L.part_begin[p]);
    const int64_t groups = (int64_t)a.n_seqs * (L.parts - 1) * a.Hv;
    int split = (int)(NUM_SMS / (groups > 0 ? groups : 1));  // CTAs per (sequence, part, head): about one wave of the SMs
    split = max(1, min(split, (part_len + 1) / 2));
    part_finish_kernel<<<dim3((unsigned)split, (unsigned)a.Hv, (unsigned)(a.n_seqs * (L.parts - 1))), FIN_THREADS, FIN_SMEM, s>>>(
        a, chunk_start, o_f32, qt_img, m0_pack, plan);
    AVE_CUDA_TRY(cudaGetLastError());
    if (beside) AVE_CUDA_TRY(cudaStreamWaitEvent(s, combined, 0));
    return AVE_GDN_OK;
  };

  SideSet* side = L.segments > 1 ? side_set(dev, stream) : nullptr;
  if (side == nullptr) {
    // one launch per pass on the caller's stream
    plan.r0 = 0; plan.rn = 1 << 24;  // every chunk (times 64 still fits an int)
    chunk_prep_kernel<<<dim3((unsigned)L.chunks, (unsigned)a.Hv), PREP_THREADS, PREP_SMEM, stream>>>(a, maps, chunk_start, po, plan, 0);
    AVE_CUDA_TRY(cudaGetLastError());
    (L.parts > 1 ? chunk_scan_tc_kernel<true> : chunk_scan_tc_kernel<false>)<<<scan_grid, SCAN_THREADS, SCAN_SMEM, stream>>>(
        a, maps, chunk_start, po.w_hi, po.w_lo, po.p_hi, po.p_lo, po.tu_hi, po.tu_lo, po.scal, o_f32, qt_img, carry, m0_pack, seq_order, plan);
    AVE_CUDA_TRY(cudaGetLastError());
    if (a.z != nullptr) {
      // packed layouts: the norm covers every row (rows of later parts are rewritten by the fix-up, which runs after it)
      const int rc = norm_rows(a, o_f32, 0, a.cu_seqlens ? a.T : part0_tokens, stream);
      if (rc != AVE_GDN_OK) return rc;
    }
    return finish_parts(stream, nullptr, nullptr, nullptr);
  }

  // Pass 1 of all ranges back to back on one helper stream, pass 2 of range i on a second once pass 1 of range i is
  // done, and (dense layouts) the gated norm of part 0's rows of range i on a third once pass 2 of range i is done; all
  // fork from the caller's stream and join back into it through events.  After an error the joins are still enqueued,
  // so that a surrounding stream capture stays well formed.
  const bool norm_per_range = a.z != nullptr && a.cu_seqlens == nullptr;
  AVE_CUDA_TRY(cudaEventRecord(side->fork, stream));
  int rc = AVE_GDN_OK;
  auto step = [&](cudaError_t e) { if (e != cudaSuccess && rc == AVE_GDN_OK) rc = cuda_fail(e); return e == cudaSuccess; };
  step(cudaStreamWaitEvent(side->prep, side->fork, 0));
  step(cudaStreamWaitEvent(side->scan, side->fork, 0));
  if (norm_per_range) step(cudaStreamWaitEvent(side->norm, side->fork, 0));
  for (int i = 0; i < L.segments && rc == AVE_GDN_OK; ++i) {
    plan.r0 = L.seg_begin[i]; plan.rn = L.seg_begin[i + 1] - L.seg_begin[i];
    if (plan.rn <= 0) continue;
    chunk_prep_kernel<<<dim3((unsigned)(a.n_seqs * L.parts * plan.rn), (unsigned)a.Hv), PREP_THREADS, PREP_SMEM, side->prep>>>(
        a, maps, chunk_start, po, plan, 1);
    if (!step(cudaGetLastError())) break;
    if (!step(cudaEventRecord(side->done[i], side->prep))) break;
    if (!step(cudaStreamWaitEvent(side->scan, side->done[i], 0))) break;
    (L.parts > 1 ? chunk_scan_tc_kernel<true> : chunk_scan_tc_kernel<false>)<<<scan_grid, SCAN_THREADS, SCAN_SMEM, side->scan>>>(
        a, maps, chunk_start, po.w_hi, po.w_lo, po.p_hi, po.p_lo, po.tu_hi, po.tu_lo, po.scal, o_f32, qt_img, carry, m0_pack, seq_order, plan);
    if (!step(cudaGetLastError())) break;
    if (norm_per_range) {
      if (!step(cudaEventRecord(side->scanned[i], side->scan))) break;
      if (!step(cudaStreamWaitEvent(side->norm, side->scanned[i], 0))) break;
      const int nrc = norm_rows(a, o_f32, min(part0_tokens, plan.r0 * C), min(part0_tokens, (plan.r0 + plan.rn) * C), side->norm);
      if (nrc != AVE_GDN_OK && rc == AVE_GDN_OK) rc = nrc;
    }
  }
  if (rc == AVE_GDN_OK) {
    if (a.z != nullptr && !norm_per_range) rc = norm_rows(a, o_f32, 0, a.T, side->scan);  // packed layout: after the last scan
    if (rc == AVE_GDN_OK) rc = finish_parts(side->scan, side->prep, side->chains_done, side->combined);
  }
  step(cudaEventRecord(side->join, side->scan));
  step(cudaStreamWaitEvent(stream, side->join, 0));
  step(cudaEventRecord(side->join_norm, norm_per_range ? side->norm : side->prep));
  step(cudaStreamWaitEvent(stream, side->join_norm, 0));
  return rc;
}

}  // namespace ave

// ------------------------------------------------------------------------------------------------ no-allocation variant
// Some callers may not allocate device memory at all: code that runs between a framework's memory-pool snapshot
// and its release (serving runtimes that hand every byte of HBM to a paged state/KV pool at start-up and forbid
// later driver allocations), plug-in callbacks that only receive pre-registered buffers, and latency-critical
// paths where an allocator call is not allowed.  For them the prefill scratch lives in this fixed array, which
// every GPU that loads the library carries until the process exits.
namespace ave {
int validate_prefill_args(const AveGdnArgs* a);
constexpr size_t kStaticScratchBytes = AVE_GDN_NOALLOC_SCRATCH_BYTES;  // 64 MiB
}
static __device__ __align__(256) unsigned char g_static_prefill_scratch[ave::kStaticScratchBytes];

// The array's name is only a host-side handle; the device address is looked up once per device (with that device
// current) and cached.  That first call on a device should be made outside any stream capture.
extern "C" int ave_gdn_chunk_prefill_noalloc(const AveGdnArgs* args, void* stream) {
  using namespace ave;
  const int rc = validate_prefill_args(args);
  if (rc != AVE_GDN_OK) return rc;
  if ((int64_t)args->B * args->T == 0 || args->n_seqs == 0) return AVE_GDN_OK;
  if (args->dk != 128 || args->dv != 128) return AVE_GDN_UNSUPPORTED;
  // the plain schedule: one launch per pass on the caller's stream, no helper streams or events, the least scratch
  if (prefill_tc_workspace_bytes(*args, true) > kStaticScratchBytes) return AVE_GDN_WORKSPACE_TOO_SMALL;
  static std::mutex mu;
  static void* scratch_of_device[64] = {};
  int dev = 0;
  AVE_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return AVE_GDN_UNSUPPORTED;
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> guard(mu);
    if (scratch_of_device[dev] == nullptr) {
      void* p = nullptr;
      AVE_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_prefill_scratch));
      scratch_of_device[dev] = p;
    }
    scratch = scratch_of_device[dev];
  }
  AveGdnArgs local = *args;
  local.workspace = scratch;
  local.workspace_bytes = kStaticScratchBytes;
  // every scratch record a launch reads is written earlier in the same launch sequence, so nothing needs clearing
  return launch_prefill_tc(local, reinterpret_cast<cudaStream_t>(stream), true);
}
