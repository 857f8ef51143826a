// Chunked gated-delta-rule prefill, fp32 CUDA-core formulation (chunk 64, WY/UT form).
//
// Two kernels share a scratch area:
//   chunk_local : one CTA per (chunk, value head), fully parallel.  Builds the in-chunk cumulative gate b,
//                 A = strict_lower(beta_i e^{b_i-b_j} k_i.k_j), solves (I+A) [W | U] = [diag(beta e^b) K | diag(beta) V]
//                 by forward substitution and forms P = lower_incl(e^{b_i-b_j} q_i.k_j).
//   chunk_scan  : one CTA per (sequence, value head, 32-column slice of dv), sequential over the chunks of
//                 the sequence with the state slice M[dk][32] held in shared memory:
//                 Vn = U - W M;  O = scale (diag(e^b) Q M + P Vn);  M <- e^{b_C} M + K^T diag(e^{b_C-b}) Vn.
// Columns of the state are independent, which is what lets one head be split over several CTAs.
#include "common.cuh"

namespace ave {

constexpr int kChunk = 64;
constexpr int kDvSlice = 32;

struct ChunkRef {
  int n;      // sequence
  int b;      // batch row
  int t0;     // first token of the chunk within the batch row
  int len;    // valid tokens (1..64)
  bool ok;
};

// Per chunk-head scratch record (floats): W[64][DK] U[64][DV] P[64][64] b[64] qn[64] kn[64]
template <int DK, int DV>
struct ScratchRec {
  static constexpr int kW = 0;
  static constexpr int kU = kW + kChunk * DK;
  static constexpr int kP = kU + kChunk * DV;
  static constexpr int kB = kP + kChunk * kChunk;
  static constexpr int kQn = kB + kChunk;
  static constexpr int kKn = kQn + kChunk;
  static constexpr int kFloats = kKn + kChunk;
};

// chunk_start[n] = number of chunks of sequences 0..n-1 (varlen only); one CTA of 1024 threads.
// The scratch is sized for T/64 + n_seqs chunks, which holds exactly when the offsets are monotone inside [0, T]; a table
// that breaks this is rejected as a whole: total = -1 (every CTA of the two passes tests it and leaves), status bit set.
__global__ void chunk_table_kernel(const int32_t* __restrict__ cu_seqlens, int n_seqs, int T, int32_t* __restrict__ chunk_start,
                                   uint32_t* __restrict__ status) {
  __shared__ int part[1024];
  const int per = (n_seqs + 1023) / 1024;
  const int lo = threadIdx.x * per, hi = min(lo + per, n_seqs);
  int s = 0, bad = 0;
  for (int n = lo; n < hi; ++n) {
    const int a0 = cu_seqlens[n], a1 = cu_seqlens[n + 1];
    bad |= (a0 < 0 || a1 < a0 || a1 > T) ? 1 : 0;
    s += max(0, (a1 - a0 + kChunk - 1) / kChunk);
  }
  part[threadIdx.x] = s;
  bad = __syncthreads_or(bad);
  if (threadIdx.x == 0) {
    int run = 0;
    for (int i = 0; i < 1024; ++i) { const int x = part[i]; part[i] = run; run += x; }
    chunk_start[n_seqs] = bad ? -1 : run;
    if (bad && status != nullptr) atomicOr(status, AVE_GDN_DEV_BAD_SEQLEN);
  }
  __syncthreads();
  if (bad) return;
  int run = part[threadIdx.x];
  for (int n = lo; n < hi; ++n) {
    chunk_start[n] = run;
    run += max(0, (cu_seqlens[n + 1] - cu_seqlens[n] + kChunk - 1) / kChunk);
  }
}

__device__ __forceinline__ ChunkRef find_chunk(const AveGdnArgs& a, const int32_t* chunk_start, int c) {
  ChunkRef r;
  r.ok = false;
  if (a.cu_seqlens == nullptr) {
    const int per = (a.T + kChunk - 1) / kChunk;
    r.n = c / per; r.b = r.n;
    if (r.n >= a.B) return r;
    r.t0 = (c - r.n * per) * kChunk;
    r.len = min(kChunk, a.T - r.t0);
    r.ok = true;
    return r;
  }
  if (c >= chunk_start[a.n_seqs]) return r;
  int lo = 0, hi = a.n_seqs;  // largest n with chunk_start[n] <= c
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (chunk_start[mid] <= c) lo = mid; else hi = mid;
  }
  const int s0 = a.cu_seqlens[lo], s1 = a.cu_seqlens[lo + 1];
  if (s0 < 0 || s1 < s0 || s1 > a.T) return r;
  r.n = lo; r.b = 0;
  r.t0 = s0 + (c - chunk_start[lo]) * kChunk;
  r.len = min(kChunk, s1 - r.t0);
  r.ok = r.len > 0;
  return r;
}

// C(i,j) = sum_d A(i,d) B(d,j) over a 256-thread CTA; thread (ti,tj) owns rows ti + a*(M/TM), cols tj + b*(N/TN).
template <int M, int N, int K, int TM, int TN, bool A_T, bool B_T, class Epi>
__device__ __forceinline__ void tile_gemm(const float* __restrict__ A, int lda, const float* __restrict__ B, int ldb, Epi epi) {
  constexpr int CT = N / TN, RT = M / TM;
  static_assert(CT * RT <= 256, "tile_gemm thread budget");
  const int tid = threadIdx.x;
  if (tid >= CT * RT) return;
  const int tj = tid % CT, ti = tid / CT;
  float acc[TM][TN];
#pragma unroll
  for (int x = 0; x < TM; ++x)
#pragma unroll
    for (int y = 0; y < TN; ++y) acc[x][y] = 0.f;
#pragma unroll 4
  for (int d = 0; d < K; ++d) {
    float av[TM], bv[TN];
#pragma unroll
    for (int x = 0; x < TM; ++x) {
      const int i = ti + x * RT;
      av[x] = A_T ? A[d * lda + i] : A[i * lda + d];
    }
#pragma unroll
    for (int y = 0; y < TN; ++y) {
      const int j = tj + y * CT;
      bv[y] = B_T ? B[j * ldb + d] : B[d * ldb + j];
    }
#pragma unroll
    for (int x = 0; x < TM; ++x)
#pragma unroll
      for (int y = 0; y < TN; ++y) acc[x][y] = fmaf(av[x], bv[y], acc[x][y]);
  }
#pragma unroll
  for (int x = 0; x < TM; ++x)
#pragma unroll
    for (int y = 0; y < TN; ++y) epi(ti + x * RT, tj + y * CT, acc[x][y], x);
}

template <int DK, int DV>
__global__ void __launch_bounds__(256) chunk_local_kernel(const AveGdnArgs a, const int32_t* __restrict__ chunk_start,
                                                          float* __restrict__ scratch) {
  using R = ScratchRec<DK, DV>;
  constexpr int LDK = DK + 1;
  extern __shared__ __align__(16) float smem[];
  float* Ks = smem;                    // [64][LDK]
  float* Qs = Ks + kChunk * LDK;       // [64][LDK]
  float* As = Qs + kChunk * LDK;       // [64][65]
  float* bs = As + kChunk * (kChunk + 1);
  float* betas = bs + kChunk;
  float* qn = betas + kChunk;
  float* kn = qn + kChunk;

  const int c = blockIdx.x, h = blockIdx.y;
  const ChunkRef cr = find_chunk(a, chunk_start, c);
  if (!cr.ok) return;
  const int hk = h / (a.Hv / a.Hk);
  const int tid = threadIdx.x;
  float* rec = scratch + ((int64_t)c * a.Hv + h) * R::kFloats;

  const __nv_bfloat16* qg = reinterpret_cast<const __nv_bfloat16*>(a.q) + cr.b * a.q_stride_b + (int64_t)hk * a.q_stride_h;
  const __nv_bfloat16* kg = reinterpret_cast<const __nv_bfloat16*>(a.k) + cr.b * a.k_stride_b + (int64_t)hk * a.k_stride_h;
  const __nv_bfloat16* vg = reinterpret_cast<const __nv_bfloat16*>(a.v) + cr.b * a.v_stride_b + (int64_t)h * a.v_stride_h;

  for (int e = tid; e < kChunk * DK; e += 256) {
    const int i = e / DK, d = e % DK;
    float kv = 0.f, qv = 0.f;
    if (i < cr.len) {
      kv = bf2f(kg[(int64_t)(cr.t0 + i) * a.k_stride_t + d]);
      qv = bf2f(qg[(int64_t)(cr.t0 + i) * a.q_stride_t + d]);
    }
    Ks[i * LDK + d] = kv;
    Qs[i * LDK + d] = qv;
  }
  if (tid < kChunk) {
    const bool valid = tid < cr.len;
    const int64_t off = cr.b * a.g_stride_b + (int64_t)(cr.t0 + tid) * a.g_stride_t + h;
    bs[tid] = valid ? a.g[off] : 0.f;
    betas[tid] = valid ? a.beta[off] : 0.f;
  }
  __syncthreads();
  if (tid == 0) {  // in-chunk cumulative gate
    float run = 0.f;
    for (int i = 0; i < kChunk; ++i) { run += bs[i]; bs[i] = run; }
  }
  if (a.flags & AVE_GDN_FLAG_QK_L2NORM) {  // 4 threads per row
    const int i = tid >> 2, part = tid & 3;
    float sk = 0.f, sq = 0.f;
    for (int d = part; d < DK; d += 4) { const float kv = Ks[i * LDK + d], qv = Qs[i * LDK + d]; sk += kv * kv; sq += qv * qv; }
    sk += __shfl_xor_sync(0xffffffffu, sk, 1); sk += __shfl_xor_sync(0xffffffffu, sk, 2);
    sq += __shfl_xor_sync(0xffffffffu, sq, 1); sq += __shfl_xor_sync(0xffffffffu, sq, 2);
    if (part == 0) { kn[i] = rsqrtf(sk + 1e-6f); qn[i] = rsqrtf(sq + 1e-6f); }
  } else if (tid < kChunk) {
    kn[tid] = 1.f; qn[tid] = 1.f;
  }
  __syncthreads();
  if (a.flags & AVE_GDN_FLAG_QK_L2NORM) {
    for (int e = tid; e < kChunk * DK; e += 256) {
      const int i = e / DK, d = e % DK;
      Ks[i * LDK + d] *= kn[i];
      Qs[i * LDK + d] *= qn[i];
    }
    __syncthreads();
  }
  if (tid < kChunk) { rec[R::kB + tid] = bs[tid]; rec[R::kQn + tid] = qn[tid]; rec[R::kKn + tid] = kn[tid]; }

  // A = strict_lower(beta_i e^{b_i-b_j} k_i.k_j) -> shared;  P = lower_incl(e^{b_i-b_j} q_i.k_j) -> scratch
  tile_gemm<kChunk, kChunk, DK, 8, 2, false, true>(Ks, LDK, Ks, LDK, [&](int i, int j, float acc, int x) {
    As[i * (kChunk + 1) + j] = (i > j) ? betas[i] * __expf(bs[i] - bs[j]) * acc : 0.f;
  });
  tile_gemm<kChunk, kChunk, DK, 8, 2, false, true>(Qs, LDK, Ks, LDK, [&](int i, int j, float acc, int x) {
    rec[R::kP + i * kChunk + j] = (i >= j) ? __expf(bs[i] - bs[j]) * acc : 0.f;
  });
  __syncthreads();

  // forward substitution, one column of [W | U] per thread
  for (int col = tid; col < DK + DV; col += 256) {
    float x[kChunk];
    const bool is_w = col < DK;
#pragma unroll
    for (int i = 0; i < kChunk; ++i) {
      float rhs;
      if (is_w) {
        rhs = betas[i] * __expf(bs[i]) * Ks[i * LDK + col];
      } else {
        rhs = (i < cr.len) ? betas[i] * bf2f(vg[(int64_t)(cr.t0 + i) * a.v_stride_t + (col - DK)]) : 0.f;
      }
#pragma unroll
      for (int j = 0; j < i; ++j) rhs = fmaf(-As[i * (kChunk + 1) + j], x[j], rhs);
      x[i] = rhs;
    }
    float* dst = is_w ? rec + R::kW + col : rec + R::kU + (col - DK);
    const int ld = is_w ? DK : DV;
#pragma unroll
    for (int i = 0; i < kChunk; ++i) dst[i * ld] = x[i];
  }
}

template <int DK, int DV>
__global__ void __launch_bounds__(256) chunk_scan_kernel(const AveGdnArgs a, const int32_t* __restrict__ chunk_start,
                                                         const float* __restrict__ scratch, float* __restrict__ o_f32) {
  using R = ScratchRec<DK, DV>;
  constexpr int NS = kDvSlice;
  extern __shared__ __align__(16) float smem[];
  float* Ws = smem;                 // [64][DK]
  float* Qs = Ws + kChunk * DK;     // [64][DK]
  float* Ks = Qs + kChunk * DK;     // [64][DK]
  float* Ps = Ks + kChunk * DK;     // [64][64]
  float* Ms = Ps + kChunk * kChunk; // [DK][NS]
  float* Vn = Ms + DK * NS;         // [64][NS]
  float* Vd = Vn + kChunk * NS;     // [64][NS]  decayed copy
  float* bs = Vd + kChunk * NS;     // [64]

  const int n = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * NS;
  const int hk = h / (a.Hv / a.Hk);
  const int tid = threadIdx.x;
  if (a.cu_seqlens != nullptr && chunk_start[a.n_seqs] < 0) return;  // the chunk table was rejected
  const SeqSpan sp = seq_span(a.cu_seqlens, n, a.T, a.status);
  if (!sp.ok) return;

  int slot = n;
  if (a.state_indices != nullptr) {
    slot = a.state_indices[n];
    if (slot >= a.num_slots) {
      if (a.status != nullptr && tid == 0) atomicOr(a.status, AVE_GDN_DEV_BAD_SLOT);
      slot = -1;
    }
  }
  __nv_bfloat16* og = reinterpret_cast<__nv_bfloat16*>(a.o) + sp.b * a.o_stride_b + (int64_t)h * a.o_stride_h;
  if (slot < 0) {  // skipped sequence: outputs are zero, no state access
    for (int e = tid; e < sp.len * NS; e += 256) {
      const int64_t tok = sp.t0 + e / NS;
      if (o_f32 != nullptr) {
        o_f32[((int64_t)sp.b * a.T + tok) * ((int64_t)a.Hv * DV) + (int64_t)h * DV + j0 + e % NS] = 0.f;
      } else {
        og[tok * a.o_stride_t + j0 + e % NS] = __float2bfloat16(0.f);
      }
    }
    return;
  }
  const int64_t tile = ((int64_t)slot * a.Hv + h) * (int64_t)(DK * DV);
  for (int e = tid; e < DK * NS; e += 256) {
    const int i = e / NS, j = e % NS;
    Ms[e] = a.initial_state ? a.initial_state[tile + (int64_t)i * DV + j0 + j] : 0.f;
  }

  const __nv_bfloat16* qg = reinterpret_cast<const __nv_bfloat16*>(a.q) + sp.b * a.q_stride_b + (int64_t)hk * a.q_stride_h;
  const __nv_bfloat16* kg = reinterpret_cast<const __nv_bfloat16*>(a.k) + sp.b * a.k_stride_b + (int64_t)hk * a.k_stride_h;
  const int n_chunks = (sp.len + kChunk - 1) / kChunk;
  const int c_first = a.cu_seqlens ? chunk_start[n] : n * ((a.T + kChunk - 1) / kChunk);

  for (int ci = 0; ci < n_chunks; ++ci) {
    const float* rec = scratch + ((int64_t)(c_first + ci) * a.Hv + h) * R::kFloats;
    const int t0 = sp.t0 + ci * kChunk;
    const int len = min(kChunk, sp.len - ci * kChunk);
    for (int e = tid; e < kChunk * DK; e += 256) {
      const int i = e / DK, d = e % DK;
      Ws[e] = rec[R::kW + e];
      float kv = 0.f, qv = 0.f;
      if (i < len) {
        kv = bf2f(kg[(int64_t)(t0 + i) * a.k_stride_t + d]) * rec[R::kKn + i];
        qv = bf2f(qg[(int64_t)(t0 + i) * a.q_stride_t + d]) * rec[R::kQn + i];
      }
      Ks[e] = kv;
      Qs[e] = qv;
    }
    for (int e = tid; e < kChunk * kChunk; e += 256) Ps[e] = rec[R::kP + e];
    if (tid < kChunk) bs[tid] = rec[R::kB + tid];
    __syncthreads();
    const float bC = bs[kChunk - 1];

    // Vn = U - W M  (and its decayed copy for the state update)
    tile_gemm<kChunk, NS, DK, 8, 1, false, false>(Ws, DK, Ms, NS, [&](int i, int j, float acc, int x) {
      const float vn = rec[R::kU + i * DV + j0 + j] - acc;
      Vn[i * NS + j] = vn;
      Vd[i * NS + j] = vn * __expf(bC - bs[i]);
    });
    // O = scale (e^{b_i} Q M + P Vn): first term kept in registers across the barrier
    float qm[8];
    tile_gemm<kChunk, NS, DK, 8, 1, false, false>(Qs, DK, Ms, NS, [&](int i, int j, float acc, int x) {
      qm[x] = acc * __expf(bs[i]);
    });
    __syncthreads();
    tile_gemm<kChunk, NS, kChunk, 8, 1, false, false>(Ps, kChunk, Vn, NS, [&](int i, int j, float acc, int x) {
      const float ov = a.scale * (qm[x] + acc);
      if (i < len) {
        if (o_f32 != nullptr) {
          o_f32[((int64_t)sp.b * a.T + t0 + i) * ((int64_t)a.Hv * DV) + (int64_t)h * DV + j0 + j] = ov;
        } else {
          og[(int64_t)(t0 + i) * a.o_stride_t + j0 + j] = __float2bfloat16(ov);
        }
      }
    });
    // M <- e^{b_C} M + K^T Vd   (each thread rewrites only the elements it owns)
    const float decay = __expf(bC);
    tile_gemm<DK, NS, kChunk, DK / 8, 1, true, false>(Ks, DK, Vd, NS, [&](int i, int j, float acc, int x) {
      Ms[i * NS + j] = decay * Ms[i * NS + j] + acc;
    });
    __syncthreads();
  }
  if (a.final_state != nullptr) {
    for (int e = tid; e < DK * NS; e += 256) {
      const int i = e / NS, j = e % NS;
      a.final_state[tile + (int64_t)i * DV + j0 + j] = Ms[e];
    }
  }
}

size_t prefill_simt_workspace_bytes(const AveGdnArgs& a) {
  const int64_t chunks = a.cu_seqlens ? (int64_t)a.T / kChunk + a.n_seqs : (int64_t)a.B * ((a.T + kChunk - 1) / kChunk);
  const int64_t rec = (a.dk == 128) ? ScratchRec<128, 128>::kFloats : ScratchRec<64, 64>::kFloats;
  size_t bytes = (((size_t)a.n_seqs + 1) * sizeof(int32_t) + 255) & ~(size_t)255;
  bytes += (size_t)chunks * a.Hv * rec * sizeof(float);
  if (a.z != nullptr) bytes += (size_t)a.B * a.T * a.Hv * a.dv * sizeof(float);
  return bytes;
}

int launch_gated_rmsnorm_f32in(const AveGdnNormArgs& a, cudaStream_t stream, const void* const* peers = nullptr, int n_peers = 0,
                               int64_t peer_off = 0);

template <int DK, int DV>
static int launch_prefill_t(const AveGdnArgs& a, cudaStream_t stream) {
  using R = ScratchRec<DK, DV>;
  const int64_t chunks = a.cu_seqlens ? (int64_t)a.T / kChunk + a.n_seqs : (int64_t)a.B * ((a.T + kChunk - 1) / kChunk);
  if (chunks == 0 || a.n_seqs == 0) return AVE_GDN_OK;
  char* ws = reinterpret_cast<char*>(a.workspace);
  int32_t* chunk_start = reinterpret_cast<int32_t*>(ws);
  size_t off = (((size_t)a.n_seqs + 1) * sizeof(int32_t) + 255) & ~(size_t)255;
  float* scratch = reinterpret_cast<float*>(ws + off);
  off += (size_t)chunks * a.Hv * R::kFloats * sizeof(float);
  float* o_f32 = a.z ? reinterpret_cast<float*>(ws + off) : nullptr;

  if (a.cu_seqlens != nullptr) chunk_table_kernel<<<1, 1024, 0, stream>>>(a.cu_seqlens, a.n_seqs, a.T, chunk_start, a.status);

  constexpr size_t smem_local = sizeof(float) * (2 * kChunk * (DK + 1) + kChunk * (kChunk + 1) + 4 * kChunk);
  constexpr size_t smem_scan = sizeof(float) * (3 * kChunk * DK + kChunk * kChunk + DK * kDvSlice + 2 * kChunk * kDvSlice + kChunk);
  static bool attr_set_dev[64] = {};  // the opt-in is per function and per device
  int dev = 0;
  AVE_CUDA_TRY(cudaGetDevice(&dev));
  bool& attr_set = attr_set_dev[dev & 63];
  if (!attr_set) {
    AVE_CUDA_TRY(cudaFuncSetAttribute(chunk_local_kernel<DK, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_local));
    AVE_CUDA_TRY(cudaFuncSetAttribute(chunk_scan_kernel<DK, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_scan));
    attr_set = true;
  }
  chunk_local_kernel<DK, DV><<<dim3((unsigned)chunks, (unsigned)a.Hv), 256, smem_local, stream>>>(a, chunk_start, scratch);
  AVE_CUDA_TRY(cudaGetLastError());
  chunk_scan_kernel<DK, DV><<<dim3((unsigned)a.n_seqs, (unsigned)a.Hv, DV / kDvSlice), 256, smem_scan, stream>>>(a, chunk_start, scratch, o_f32);
  AVE_CUDA_TRY(cudaGetLastError());
  if (a.z != nullptr) {
    AveGdnNormArgs na{};
    na.struct_size = sizeof(na);
    na.flags = a.flags & AVE_GDN_FLAG_GATE_FIRST;
    na.x = o_f32; na.z = a.z; na.weight = a.norm_weight; na.y = a.o;
    na.d = DV; na.heads = a.Hv; na.eps = a.norm_eps;
    na.x_stride_t = (int64_t)a.Hv * DV; na.x_stride_h = DV;
    // the norm kernel indexes rows as (token, head); batches are folded in one launch per batch row
    for (int b = 0; b < a.B; ++b) {
      AveGdnNormArgs nb = na;
      nb.rows = (int64_t)a.T * a.Hv;
      nb.x = o_f32 + (int64_t)b * a.T * a.Hv * DV;
      nb.z = reinterpret_cast<const __nv_bfloat16*>(a.z) + b * a.z_stride_b;
      nb.y = reinterpret_cast<__nv_bfloat16*>(a.o) + b * a.o_stride_b;
      nb.z_stride_t = a.z_stride_t; nb.z_stride_h = a.z_stride_h;
      nb.y_stride_t = a.o_stride_t; nb.y_stride_h = a.o_stride_h;
      const int rc = launch_gated_rmsnorm_f32in(nb, stream);
      if (rc != AVE_GDN_OK) return rc;
    }
  }
  return AVE_GDN_OK;
}

int launch_prefill_simt(const AveGdnArgs& a, cudaStream_t stream) {
  if (a.dk == 128 && a.dv == 128) return launch_prefill_t<128, 128>(a, stream);
  if (a.dk == 64 && a.dv == 64) return launch_prefill_t<64, 64>(a, stream);
  return AVE_GDN_UNSUPPORTED;
}

}  // namespace ave
