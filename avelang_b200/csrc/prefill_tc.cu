// Chunked gated-delta-rule prefill on the tensor cores (d_k = d_v = 128, chunk 64).
//
// Pass 1, chunk_prep (one CTA per (chunk, value head), fully parallel): in-chunk cumulative gate b,
//   A = strict_lower(beta_i e^{b_i-b_j} k_i.k_j), forward substitution for W = (I+A)^-1 diag(beta e^b) K and
//   U = (I+A)^-1 diag(beta) V, P = lower_incl(e^{b_i-b_j} q_i.k_j).  W and P leave as bf16 hi+lo pairs (the
//   tensor cores then see 16 significant bits), U as fp32, plus per-token scale vectors.
// Pass 2, chunk_scan (one CTA per (sequence, value head)): the recurrence over chunks with the state kept
//   on chip, transposed (H = M^T, rows = d_v = TMEM lanes) so that every MMA has M = 128:
//     Vn^T = U^T - H W^T                 (A = H hi/lo from TMEM, B = W hi/lo, K-major)
//     O^T  = diag-scaled H Q^T + Vn^T P^T (A = H or Vn hi/lo from TMEM, B = Q or P hi/lo, K-major)
//     H   <- e^{b_C} H + Vd^T K          (A = Vd hi/lo from TMEM, B = K, MN-major), Vd_j = e^{b_C-b_j} Vn_j
//   fp32 master copy of H lives in the epilogue threads' registers; its bf16 hi/lo image is rewritten to TMEM
//   every chunk.  Warp roles: 0 = TMA loader, 1 = MMA issuer, 2..9 = two epilogue groups (each covers all
//   128 TMEM lanes and half of the columns).  All waits are bounded; on give-up the CTA drains and sets a
//   status bit.
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
  __nv_bfloat16 *w_hi, *w_lo, *p_hi, *p_lo;
  float *u, *scal;
};

struct ChunkRef { int n, b, t0, len; bool ok; };

__device__ __forceinline__ ChunkRef find_chunk(const AveGdnArgs& a, const int32_t* chunk_start, int c) {
  ChunkRef r; r.ok = false;
  if (a.cu_seqlens == nullptr) {
    const int per = (a.T + C - 1) / C;
    r.n = c / per; r.b = r.n;
    if (r.n >= a.B) return r;
    r.t0 = (c - r.n * per) * C; r.len = min(C, a.T - r.t0); r.ok = true;
    return r;
  }
  if (c >= chunk_start[a.n_seqs]) return r;
  int lo = 0, hi = a.n_seqs;
  while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (chunk_start[mid] <= c) lo = mid; else hi = mid; }
  const int s0 = a.cu_seqlens[lo], s1 = a.cu_seqlens[lo + 1];
  if (s0 < 0 || s1 < s0 || s1 > a.T) return r;
  r.n = lo; r.b = 0; r.t0 = s0 + (c - chunk_start[lo]) * C; r.len = min(C, s1 - r.t0); r.ok = r.len > 0;
  return r;
}

__global__ void chunk_table_tc_kernel(const int32_t* __restrict__ cu_seqlens, int n_seqs, int32_t* __restrict__ chunk_start) {
  __shared__ int part[1024];
  const int per = (n_seqs + 1023) / 1024;
  const int lo = threadIdx.x * per, hi = min(lo + per, n_seqs);
  int s = 0;
  for (int n = lo; n < hi; ++n) s += max(0, (cu_seqlens[n + 1] - cu_seqlens[n] + C - 1) / C);
  part[threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int i = 0; i < 1024; ++i) { const int x = part[i]; part[i] = run; run += x; }
    chunk_start[n_seqs] = run;
  }
  __syncthreads();
  int run = part[threadIdx.x];
  for (int n = lo; n < hi; ++n) { chunk_start[n] = run; run += max(0, (cu_seqlens[n + 1] - cu_seqlens[n] + C - 1) / C); }
}

__device__ __forceinline__ void split_bf16(float x, __nv_bfloat16& hi, __nv_bfloat16& lo) {
  hi = __float2bfloat16(x);
  lo = __float2bfloat16(x - __bfloat162float(hi));
}

// 64x64 = A(64xD) * B(64xD)^T over a 256-thread CTA, both operands row-major with leading dimension ld.
template <class Epi>
__device__ __forceinline__ void gram64(const float* __restrict__ A, const float* __restrict__ B, int ld, Epi epi) {
  const int tid = threadIdx.x, tj = tid % 32, ti = tid / 32;
  float acc[8][2];
#pragma unroll
  for (int x = 0; x < 8; ++x) { acc[x][0] = 0.f; acc[x][1] = 0.f; }
#pragma unroll 4
  for (int d = 0; d < D; ++d) {
    const float b0 = B[tj * ld + d], b1 = B[(tj + 32) * ld + d];
#pragma unroll
    for (int x = 0; x < 8; ++x) {
      const float av = A[(ti + x * 8) * ld + d];
      acc[x][0] = fmaf(av, b0, acc[x][0]);
      acc[x][1] = fmaf(av, b1, acc[x][1]);
    }
  }
#pragma unroll
  for (int x = 0; x < 8; ++x) { epi(ti + x * 8, tj, acc[x][0]); epi(ti + x * 8, tj + 32, acc[x][1]); }
}

__global__ void __launch_bounds__(256) chunk_prep_kernel(const AveGdnArgs a, const int32_t* __restrict__ chunk_start, PrepOut out) {
  constexpr int LDK = D + 1;
  extern __shared__ __align__(16) float smem_f[];
  float* Ks = smem_f;
  float* Qs = Ks + C * LDK;
  float* As = Qs + C * LDK;      // [64][65]
  float* bs = As + C * (C + 1);
  float* betas = bs + C;
  float* qn = betas + C;
  float* kn = qn + C;

  const int c = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const ChunkRef cr = find_chunk(a, chunk_start, c);
  if (!cr.ok) return;
  const int hk = h / (a.Hv / a.Hk);
  const int64_t rec = (int64_t)c * a.Hv + h;
  const __nv_bfloat16* qg = reinterpret_cast<const __nv_bfloat16*>(a.q) + cr.b * a.q_stride_b + (int64_t)hk * a.q_stride_h;
  const __nv_bfloat16* kg = reinterpret_cast<const __nv_bfloat16*>(a.k) + cr.b * a.k_stride_b + (int64_t)hk * a.k_stride_h;
  const __nv_bfloat16* vg = reinterpret_cast<const __nv_bfloat16*>(a.v) + cr.b * a.v_stride_b + (int64_t)h * a.v_stride_h;

  for (int e = tid; e < C * D; e += 256) {
    const int i = e / D, d = e % D;
    float kv = 0.f, qv = 0.f;
    if (i < cr.len) {
      kv = bf2f(kg[(int64_t)(cr.t0 + i) * a.k_stride_t + d]);
      qv = bf2f(qg[(int64_t)(cr.t0 + i) * a.q_stride_t + d]);
    }
    Ks[i * LDK + d] = kv; Qs[i * LDK + d] = qv;
  }
  if (tid < C) {
    const bool valid = tid < cr.len;
    const int64_t off = cr.b * a.g_stride_b + (int64_t)(cr.t0 + tid) * a.g_stride_t + h;
    bs[tid] = valid ? a.g[off] : 0.f;
    betas[tid] = valid ? a.beta[off] : 0.f;
  }
  __syncthreads();
  if (tid == 0) { float run = 0.f; for (int i = 0; i < C; ++i) { run += bs[i]; bs[i] = run; } }
  if (a.flags & AVE_GDN_FLAG_QK_L2NORM) {
    const int i = tid >> 2, part = tid & 3;
    float sk = 0.f, sq = 0.f;
    for (int d = part; d < D; d += 4) { const float kv = Ks[i * LDK + d], qv = Qs[i * LDK + d]; sk += kv * kv; sq += qv * qv; }
    sk += __shfl_xor_sync(0xffffffffu, sk, 1); sk += __shfl_xor_sync(0xffffffffu, sk, 2);
    sq += __shfl_xor_sync(0xffffffffu, sq, 1); sq += __shfl_xor_sync(0xffffffffu, sq, 2);
    if (part == 0) { kn[i] = rsqrtf(sk + 1e-6f); qn[i] = rsqrtf(sq + 1e-6f); }
  } else if (tid < C) { kn[tid] = 1.f; qn[tid] = 1.f; }
  __syncthreads();
  const float bC = bs[C - 1];
  if (tid < C) {
    float* sc = out.scal + rec * SCAL_FLOATS;
    sc[tid] = __expf(bs[tid]) * qn[tid];             // o_i = scale (qs_i (H q_i) + ...)
    sc[C + tid] = __expf(bC - bs[tid]) * kn[tid];    // Vd_j = ks_j Vn_j
    sc[2 * C + tid] = __expf(bC);
  }
  // A (normalised k) -> shared;  P (normalised q, k) -> bf16 hi/lo
  gram64(Ks, Ks, LDK, [&](int i, int j, float acc) {
    As[i * (C + 1) + j] = (i > j) ? betas[i] * __expf(bs[i] - bs[j]) * acc * kn[i] * kn[j] : 0.f;
  });
  {
    __nv_bfloat16* ph = out.p_hi + rec * (C * C);
    __nv_bfloat16* pl = out.p_lo + rec * (C * C);
    gram64(Qs, Ks, LDK, [&](int i, int j, float acc) {
      const float p = (i >= j) ? __expf(bs[i] - bs[j]) * acc * qn[i] * kn[j] : 0.f;
      __nv_bfloat16 hi, lo;
      split_bf16(p, hi, lo);
      ph[i * C + j] = hi; pl[i * C + j] = lo;
    });
  }
  __syncthreads();
  // forward substitution, one column of [W | U] per thread
  {
    const int col = tid;
    const bool is_w = col < D;
    float x[C];
#pragma unroll
    for (int i = 0; i < C; ++i) {
      float rhs;
      if (is_w) rhs = betas[i] * __expf(bs[i]) * kn[i] * Ks[i * LDK + col];
      else rhs = (i < cr.len) ? betas[i] * bf2f(vg[(int64_t)(cr.t0 + i) * a.v_stride_t + (col - D)]) : 0.f;
#pragma unroll
      for (int j = 0; j < i; ++j) rhs = fmaf(-As[i * (C + 1) + j], x[j], rhs);
      x[i] = rhs;
    }
    if (is_w) {
      __nv_bfloat16* wh = out.w_hi + rec * (C * D) + col;
      __nv_bfloat16* wl = out.w_lo + rec * (C * D) + col;
#pragma unroll
      for (int i = 0; i < C; ++i) { __nv_bfloat16 hi, lo; split_bf16(x[i], hi, lo); wh[i * D] = hi; wl[i * D] = lo; }
    } else {
      float* u = out.u + rec * (C * D) + (col - D);
#pragma unroll
      for (int i = 0; i < C; ++i) u[i * D] = x[i];
    }
  }
}

// ------------------------------------------------------------------------------------------------ pass 2
constexpr int SCAN_THREADS = 320;
constexpr int ST_WHI = 0, ST_WLO = 16384, ST_Q = 32768, ST_K = 49152, ST_PHI = 65536, ST_PLO = 73728, ST_SCAL = 81920;
constexpr int STAGE = 82944;                         // multiple of 1024
constexpr uint32_t STAGE_TX = 4 * 16384 + 2 * 8192 + SCAL_FLOATS * 4;
constexpr int OFF_STAGING = 2 * STAGE;               // fp32 [64][128]
constexpr int OFF_BARS = OFF_STAGING + C * D * 4;
constexpr size_t SCAN_SMEM = OFF_BARS + 256 + 1024;
// TMEM columns
constexpr uint32_t TM_HHI = 0, TM_HLO = 64, TM_VN = 128, TM_VNHI = 128, TM_VNLO = 160, TM_VDHI = 192, TM_VDLO = 224,
                   TM_O1 = 256, TM_O2 = 320, TM_DH = 384;

struct ScanMaps {
  CUtensorMap q, k, w_hi, w_lo, p_hi, p_lo;
};

__device__ __forceinline__ uint32_t pack_hi(float x0, float x1) { return pack_bf16x2(x0, x1); }
__device__ __forceinline__ uint32_t pack_lo(float x0, float x1, uint32_t hi_packed) {
  const float h0 = __uint_as_float(hi_packed << 16), h1 = __uint_as_float(hi_packed & 0xffff0000u);
  return pack_bf16x2(x0 - h0, x1 - h1);
}
// Barrier among the 8 epilogue warps built on an mbarrier so that, unlike bar.sync, the wait is bounded.
__device__ __forceinline__ bool epi_sync(uint64_t* bar, uint32_t& phase, int lane, volatile uint32_t* abort_flag) {
  __syncwarp();
  if (lane == 0) tc::mbar_arrive(bar);
  const bool ok = tc::mbar_wait(bar, phase, abort_flag);
  phase ^= 1u;
  return ok;
}

__global__ void __launch_bounds__(SCAN_THREADS, 1)
chunk_scan_tc_kernel(const AveGdnArgs a, const __grid_constant__ ScanMaps maps, const int32_t* __restrict__ chunk_start,
                     const float* __restrict__ u_ws, const float* __restrict__ scal_ws) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  float* staging = reinterpret_cast<float*>(smem + OFF_STAGING);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BARS);
  uint64_t* full = bars;          // [2]
  uint64_t* empty = bars + 2;     // [2]
  uint64_t* h_ready = bars + 4;
  uint64_t* vn_full = bars + 5;
  uint64_t* vn_ready = bars + 6;
  uint64_t* dh_full = bars + 7;
  uint64_t* o_full = bars + 8;
  uint64_t* o_empty = bars + 9;
  uint64_t* epi_bar = bars + 10;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x / a.Hv, h = blockIdx.x % a.Hv;
  const int hk = h / (a.Hv / a.Hk);
  const SeqSpan sp = seq_span(a.cu_seqlens, n, a.T, a.status);
  if (!sp.ok || sp.len == 0) {
    // zero-length sequence: the final state is the initial state
    if (sp.ok && a.final_state != nullptr && a.final_state != a.initial_state) {
      int slot = a.state_indices ? a.state_indices[n] : n;
      if (slot >= 0 && slot < a.num_slots) {
        const int64_t tile = ((int64_t)slot * a.Hv + h) * (int64_t)(D * D);
        for (int e = threadIdx.x; e < D * D; e += SCAN_THREADS)
          a.final_state[tile + e] = a.initial_state ? a.initial_state[tile + e] : 0.f;
      }
    }
    return;
  }
  int slot = n;
  if (a.state_indices != nullptr) {
    slot = a.state_indices[n];
    if (slot >= a.num_slots) {
      if (a.status != nullptr && threadIdx.x == 0) atomicOr(a.status, AVE_GDN_DEV_BAD_SLOT);
      slot = -1;
    }
  }
  __nv_bfloat16* og = reinterpret_cast<__nv_bfloat16*>(a.o) + sp.b * a.o_stride_b + (int64_t)h * a.o_stride_h;
  if (slot < 0) {
    for (int e = threadIdx.x; e < sp.len * D; e += SCAN_THREADS)
      og[(int64_t)(sp.t0 + e / D) * a.o_stride_t + e % D] = __float2bfloat16(0.f);
    return;
  }
  const int n_chunks = (sp.len + C - 1) / C;
  const int c_first = a.cu_seqlens ? chunk_start[n] : n * ((a.T + C - 1) / C);

  if (threadIdx.x == 0) {
    tc::mbar_init(&full[0], 1); tc::mbar_init(&full[1], 1);
    tc::mbar_init(&empty[0], 9); tc::mbar_init(&empty[1], 9);
    tc::mbar_init(h_ready, 8); tc::mbar_init(vn_full, 1); tc::mbar_init(vn_ready, 8);
    tc::mbar_init(dh_full, 1); tc::mbar_init(o_full, 1); tc::mbar_init(o_empty, 8);
    tc::mbar_init(epi_bar, 8);
    *abort_flag = 0;
    tc::fence_barrier_init();
  }
  if (warp == 1) tc::tmem_alloc(tmem_slot, 512);
  tc::tc_fence_before_sync();
  __syncthreads();
  tc::tc_fence_after_sync();
  const uint32_t tm = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ loader
    if (lane == 0) {
      for (int c = 0; c < n_chunks; ++c) {
        const int s = c & 1;
        const uint32_t u = (uint32_t)(c >> 1);
        if (!tc::mbar_wait(&empty[s], (u & 1u) ^ 1u, abort_flag)) break;
        uint8_t* st = smem + s * STAGE;
        const int64_t rec = (int64_t)(c_first + c) * a.Hv + h;
        const int row = (int)(rec * C);
        const int tok = sp.t0 + c * C;
        tc::mbar_expect_tx(&full[s], STAGE_TX);
        tc::tma_load_2d(st + ST_WHI, &maps.w_hi, &full[s], 0, row);
        tc::tma_load_2d(st + ST_WHI + 8192, &maps.w_hi, &full[s], 64, row);
        tc::tma_load_2d(st + ST_WLO, &maps.w_lo, &full[s], 0, row);
        tc::tma_load_2d(st + ST_WLO + 8192, &maps.w_lo, &full[s], 64, row);
        tc::tma_load_4d(st + ST_Q, &maps.q, &full[s], 0, hk, tok, sp.b);
        tc::tma_load_4d(st + ST_Q + 8192, &maps.q, &full[s], 64, hk, tok, sp.b);
        tc::tma_load_4d(st + ST_K, &maps.k, &full[s], 0, hk, tok, sp.b);
        tc::tma_load_4d(st + ST_K + 8192, &maps.k, &full[s], 64, hk, tok, sp.b);
        tc::tma_load_2d(st + ST_PHI, &maps.p_hi, &full[s], 0, row);
        tc::tma_load_2d(st + ST_PLO, &maps.p_lo, &full[s], 0, row);
        tc::bulk_load(st + ST_SCAL, scal_ws + rec * SCAL_FLOATS, SCAL_FLOATS * 4, &full[s]);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t id_vn = tc::idesc_f16(128, 64, 1, 1, false, false, true, false);   // negated A
      constexpr uint32_t id_n64 = tc::idesc_f16(128, 64, 1, 1, false, false);
      constexpr uint32_t id_dh = tc::idesc_f16(128, 128, 1, 1, false, true);                // B MN-major
      for (int c = 0; c < n_chunks; ++c) {
        const int s = c & 1;
        const uint32_t cp = (uint32_t)c & 1u, u = (uint32_t)(c >> 1);
        const uint32_t sb = tc::smem_u32(smem + s * STAGE);
        if (!tc::mbar_wait(&full[s], u & 1u, abort_flag)) break;
        if (!tc::mbar_wait(h_ready, cp, abort_flag)) break;
        tc::tc_fence_after_sync();
        // Vn^T accumulator = -(Hhi Whi^T + Hlo Whi^T + Hhi Wlo^T)
#pragma unroll
        for (int t = 0; t < 3; ++t) {
          const uint32_t a_col = (t == 1) ? TM_HLO : TM_HHI;
          const uint32_t b_base = sb + ((t == 2) ? ST_WLO : ST_WHI);
#pragma unroll
          for (int k = 0; k < 8; ++k)
            tc::mma_ts(tm + TM_VN, tm + a_col + 8 * k, tc::smem_desc_sw128(b_base + (k >> 2) * 8192 + (k & 3) * 32, 16, 1024), id_vn,
                       (t | k) != 0 ? 1u : 0u);
        }
        tc::mma_commit(vn_full);
        if (!tc::mbar_wait(o_empty, cp ^ 1u, abort_flag)) break;
        tc::tc_fence_after_sync();
        // O1 = (Hhi + Hlo) Q^T
#pragma unroll
        for (int t = 0; t < 2; ++t) {
#pragma unroll
          for (int k = 0; k < 8; ++k)
            tc::mma_ts(tm + TM_O1, tm + (t ? TM_HLO : TM_HHI) + 8 * k,
                       tc::smem_desc_sw128(sb + ST_Q + (k >> 2) * 8192 + (k & 3) * 32, 16, 1024), id_n64, (t | k) != 0 ? 1u : 0u);
        }
        if (!tc::mbar_wait(vn_ready, cp, abort_flag)) break;
        tc::tc_fence_after_sync();
        // dH = (Vd_hi + Vd_lo)^T-contracted with K over the chunk's tokens
#pragma unroll
        for (int t = 0; t < 2; ++t) {
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc::mma_ts(tm + TM_DH, tm + (t ? TM_VDLO : TM_VDHI) + 8 * k, tc::smem_desc_sw128(sb + ST_K + k * 2048, 8192, 1024), id_dh,
                       (t | k) != 0 ? 1u : 0u);
        }
        tc::mma_commit(dh_full);
        // O2 = Vn_hi Phi^T + Vn_lo Phi^T + Vn_hi Plo^T
#pragma unroll
        for (int t = 0; t < 3; ++t) {
          const uint32_t a_col = (t == 1) ? TM_VNLO : TM_VNHI;
          const uint32_t b_base = sb + ((t == 2) ? ST_PLO : ST_PHI);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc::mma_ts(tm + TM_O2, tm + a_col + 8 * k, tc::smem_desc_sw128(b_base + k * 32, 16, 1024), id_n64, (t | k) != 0 ? 1u : 0u);
        }
        tc::mma_commit(o_full);
        tc::mma_commit(&empty[s]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue groups
    const int ew = warp - 2;            // 0..7
    const int grp = ew >> 2;            // column half
    const int quarter = warp & 3;       // TMEM lane quarter this warp may touch
    const int d = quarter * 32 + lane;  // row of H (d_v index)
    const uint32_t lane_addr = tm + ((uint32_t)(quarter * 32) << 16);
    const int64_t tile = ((int64_t)slot * a.Hv + h) * (int64_t)(D * D);
    bool alive = true;
    uint32_t epi_phase = 0;

    float Hreg[64];  // H[d][64*grp + i] = M[64*grp + i][d]
    if (a.initial_state != nullptr) {
#pragma unroll
      for (int i = 0; i < 64; ++i) Hreg[i] = a.initial_state[tile + (int64_t)(64 * grp + i) * D + d];
    } else {
#pragma unroll
      for (int i = 0; i < 64; ++i) Hreg[i] = 0.f;
    }
    auto publish_h = [&]() {
      uint32_t hi[32], lo[32];
#pragma unroll
      for (int w = 0; w < 32; ++w) {
        hi[w] = pack_hi(Hreg[2 * w], Hreg[2 * w + 1]);
        lo[w] = pack_lo(Hreg[2 * w], Hreg[2 * w + 1], hi[w]);
      }
      tc::tmem_st32(lane_addr + TM_HHI + 32 * grp, hi);
      tc::tmem_st32(lane_addr + TM_HLO + 32 * grp, lo);
      tc::tmem_st_wait();
      tc::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) tc::mbar_arrive(h_ready);
    };
    publish_h();

    for (int c = 0; c < n_chunks && alive; ++c) {
      const int s = c & 1;
      const uint32_t cp = (uint32_t)c & 1u, u = (uint32_t)(c >> 1);
      const int64_t rec = (int64_t)(c_first + c) * a.Hv + h;
      const float* scal = reinterpret_cast<const float*>(smem + s * STAGE + ST_SCAL);
      const int len = min(C, sp.len - c * C);
      // U^T for this thread's row and token half, fetched before the accumulator is ready
      float uv[32];
      {
        const float* up = u_ws + rec * (C * D) + (int64_t)(32 * grp) * D + d;
#pragma unroll
        for (int j = 0; j < 32; ++j) uv[j] = __ldg(up + j * D);
      }
      if (!tc::mbar_wait(&full[s], u & 1u, abort_flag)) { alive = false; break; }
      if (!tc::mbar_wait(vn_full, cp, abort_flag)) { alive = false; break; }
      tc::tc_fence_after_sync();
      {
        uint32_t acc[32];
        tc::tmem_ld32(lane_addr + TM_VN + 32 * grp, acc);
        tc::tmem_ld_wait();
        // both groups have read the accumulator before its columns are reused
        if (!epi_sync(epi_bar, epi_phase, lane, abort_flag)) { alive = false; break; }
        uint32_t vh[16], vl[16], dh[16], dl[16];
#pragma unroll
        for (int w = 0; w < 16; ++w) {
          const float v0 = uv[2 * w] + __uint_as_float(acc[2 * w]);
          const float v1 = uv[2 * w + 1] + __uint_as_float(acc[2 * w + 1]);
          vh[w] = pack_hi(v0, v1);
          vl[w] = pack_lo(v0, v1, vh[w]);
          const float e0 = v0 * scal[C + 32 * grp + 2 * w], e1 = v1 * scal[C + 32 * grp + 2 * w + 1];
          dh[w] = pack_hi(e0, e1);
          dl[w] = pack_lo(e0, e1, dh[w]);
        }
        tc::tmem_st16(lane_addr + TM_VNHI + 16 * grp, vh);
        tc::tmem_st16(lane_addr + TM_VNLO + 16 * grp, vl);
        tc::tmem_st16(lane_addr + TM_VDHI + 16 * grp, dh);
        tc::tmem_st16(lane_addr + TM_VDLO + 16 * grp, dl);
        tc::tmem_st_wait();
        tc::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(vn_ready);
      }
      // state update
      if (!tc::mbar_wait(dh_full, cp, abort_flag)) { alive = false; break; }
      tc::tc_fence_after_sync();
      {
        const float decay = scal[2 * C];
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t dh[32];
          tc::tmem_ld32(lane_addr + TM_DH + 64 * grp + 32 * half, dh);
          tc::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) Hreg[32 * half + i] = fmaf(decay, Hreg[32 * half + i], __uint_as_float(dh[i]));
        }
        publish_h();
      }
      // output
      if (!tc::mbar_wait(o_full, cp, abort_flag)) { alive = false; break; }
      tc::tc_fence_after_sync();
      {
        uint32_t o1[32], o2[32];
        tc::tmem_ld32(lane_addr + TM_O1 + 32 * grp, o1);
        tc::tmem_ld32(lane_addr + TM_O2 + 32 * grp, o2);
        tc::tmem_ld_wait();
        tc::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) tc::mbar_arrive(o_empty);
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int i = 32 * grp + j;
          staging[i * D + d] = a.scale * fmaf(scal[i], __uint_as_float(o1[j]), __uint_as_float(o2[j]));
        }
      }
      if (!epi_sync(epi_bar, epi_phase, lane, abort_flag)) { alive = false; break; }
      {
        const bool gate_first = (a.flags & AVE_GDN_FLAG_GATE_FIRST) != 0;
#pragma unroll 1
        for (int r = 0; r < 8; ++r) {
          const int i = ew * 8 + r;
          if (i >= len) break;
          const int64_t tok = sp.t0 + c * C + i;
          float4 ov = *reinterpret_cast<const float4*>(staging + i * D + 4 * lane);
          float o4[4] = {ov.x, ov.y, ov.z, ov.w};
          if (a.z != nullptr) {
            float zz[4];
            unpack_bf16x4(*reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(a.z) + sp.b * a.z_stride_b +
                                                          tok * a.z_stride_t + (int64_t)h * a.z_stride_h + 4 * lane), zz);
            if (gate_first) {
#pragma unroll
              for (int e = 0; e < 4; ++e) o4[e] *= silu(zz[e]);
            }
            const float ss = warp_sum(o4[0] * o4[0] + o4[1] * o4[1] + o4[2] * o4[2] + o4[3] * o4[3]);
            const float rinv = rsqrtf(ss * (1.0f / D) + a.norm_eps);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float w = a.norm_weight ? a.norm_weight[4 * lane + e] : 1.0f;
              o4[e] = o4[e] * rinv * w * (gate_first ? 1.0f : silu(zz[e]));
            }
          }
          *reinterpret_cast<uint2*>(og + tok * a.o_stride_t + 4 * lane) = make_uint2(pack_bf16x2(o4[0], o4[1]), pack_bf16x2(o4[2], o4[3]));
        }
      }
      // staging may be overwritten by the next chunk
      if (!epi_sync(epi_bar, epi_phase, lane, abort_flag)) { alive = false; break; }
      if (lane == 0) tc::mbar_arrive(&empty[s]);
    }
    if (alive && a.final_state != nullptr) {
#pragma unroll
      for (int i = 0; i < 64; ++i) a.final_state[tile + (int64_t)(64 * grp + i) * D + d] = Hreg[i];
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

struct WsLayout {
  size_t chunk_start, w_hi, w_lo, p_hi, p_lo, u, scal, total;
  int64_t chunks;
};

WsLayout ws_layout(const AveGdnArgs& a) {
  WsLayout L;
  L.chunks = a.cu_seqlens ? (int64_t)a.T / C + a.n_seqs : (int64_t)a.B * ((a.T + C - 1) / C);
  const size_t recs = (size_t)L.chunks * a.Hv;
  auto up = [](size_t x) { return (x + 1023) & ~(size_t)1023; };
  size_t off = 0;
  L.chunk_start = off; off = up(off + ((size_t)a.n_seqs + 1) * 4);
  L.w_hi = off; off = up(off + recs * REC_W);
  L.w_lo = off; off = up(off + recs * REC_W);
  L.p_hi = off; off = up(off + recs * REC_P);
  L.p_lo = off; off = up(off + recs * REC_P);
  L.u = off; off = up(off + recs * (size_t)(C * D * 4));
  L.scal = off; off = up(off + recs * (size_t)(SCAL_FLOATS * 4));
  L.total = off;
  return L;
}

}  // namespace

size_t prefill_tc_workspace_bytes(const AveGdnArgs& a) { return ws_layout(a).total; }

int launch_prefill_tc(const AveGdnArgs& a, cudaStream_t stream) {
  const WsLayout L = ws_layout(a);
  if (L.chunks == 0 || a.n_seqs == 0) return AVE_GDN_OK;
  char* ws = reinterpret_cast<char*>(a.workspace);
  int32_t* chunk_start = reinterpret_cast<int32_t*>(ws + L.chunk_start);
  PrepOut po;
  po.w_hi = reinterpret_cast<__nv_bfloat16*>(ws + L.w_hi);
  po.w_lo = reinterpret_cast<__nv_bfloat16*>(ws + L.w_lo);
  po.p_hi = reinterpret_cast<__nv_bfloat16*>(ws + L.p_hi);
  po.p_lo = reinterpret_cast<__nv_bfloat16*>(ws + L.p_lo);
  po.u = reinterpret_cast<float*>(ws + L.u);
  po.scal = reinterpret_cast<float*>(ws + L.scal);

  ScanMaps maps;
  const uint64_t rows = (uint64_t)L.chunks * a.Hv * C;
  {
    const uint64_t dw[2] = {D, rows}, sw[2] = {2, D * 2}, dp[2] = {C, rows}, spp[2] = {2, C * 2};
    const uint32_t box[2] = {64, 64};
    int rc;
    if ((rc = make_tmap(&maps.w_hi, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, po.w_hi, 2, dw, sw, box, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
    if ((rc = make_tmap(&maps.w_lo, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, po.w_lo, 2, dw, sw, box, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
    if ((rc = make_tmap(&maps.p_hi, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, po.p_hi, 2, dp, spp, box, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
    if ((rc = make_tmap(&maps.p_lo, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, po.p_lo, 2, dp, spp, box, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
    const uint32_t box4[4] = {64, 1, 64, 1};
    const uint64_t dq[4] = {D, (uint64_t)a.Hk, (uint64_t)a.T, (uint64_t)a.B};
    const uint64_t sq[4] = {2, (uint64_t)a.q_stride_h * 2, (uint64_t)a.q_stride_t * 2, (uint64_t)(a.B > 1 ? a.q_stride_b : a.q_stride_t * a.T) * 2};
    const uint64_t sk[4] = {2, (uint64_t)a.k_stride_h * 2, (uint64_t)a.k_stride_t * 2, (uint64_t)(a.B > 1 ? a.k_stride_b : a.k_stride_t * a.T) * 2};
    if ((rc = make_tmap(&maps.q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(a.q), 4, dq, sq, box4, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
    if ((rc = make_tmap(&maps.k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(a.k), 4, dq, sk, box4, CU_TENSOR_MAP_SWIZZLE_128B))) return rc;
  }

  if (a.cu_seqlens != nullptr) chunk_table_tc_kernel<<<1, 1024, 0, stream>>>(a.cu_seqlens, a.n_seqs, chunk_start);
  constexpr size_t smem_prep = sizeof(float) * (2 * C * (D + 1) + C * (C + 1) + 4 * C);
  static bool attr_set_dev[64] = {};
  int dev = 0;
  AVE_CUDA_TRY(cudaGetDevice(&dev));
  if (!attr_set_dev[dev & 63]) {
    AVE_CUDA_TRY(cudaFuncSetAttribute(chunk_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_prep));
    AVE_CUDA_TRY(cudaFuncSetAttribute(chunk_scan_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SCAN_SMEM));
    attr_set_dev[dev & 63] = true;
  }
  chunk_prep_kernel<<<dim3((unsigned)L.chunks, (unsigned)a.Hv), 256, smem_prep, stream>>>(a, chunk_start, po);
  AVE_CUDA_TRY(cudaGetLastError());
  chunk_scan_tc_kernel<<<(unsigned)a.n_seqs * (unsigned)a.Hv, SCAN_THREADS, SCAN_SMEM, stream>>>(a, maps, chunk_start, po.u, po.scal);
  AVE_CUDA_TRY(cudaGetLastError());
  return AVE_GDN_OK;
}

}  // namespace ave
