// Fused recurrent gated-delta-rule step ("decode"): one CTA per (sequence, value head).
//
// The fp32 state tile M[dk][dv] is streamed from HBM into registers once with 128-bit loads, both
// column reductions (r = M^T k, p = M^T q) are taken in the same sweep over the old state, and
//     u = beta (v - a r),   o = scale (a p + u (k.q)),   M <- a M + k u^T,   a = exp(g)
// is applied in registers before the tile is streamed back to the same slot.  One read and one
// write of the state per token; for T > 1 the tile stays in registers across the tokens.
#include "common.cuh"
#include "tc.cuh"

namespace ave {

template <int DK, int DV>
struct DecodeCfg {
  static constexpr int kThreads = 256;
  static constexpr int kWarps = 8;
  static constexpr int kLanesPerRow = DV / 4;             // one float4 per lane
  static constexpr int kRowsPerLoad = 32 / kLanesPerRow;  // rows covered by one warp-wide load
  static constexpr int kRowsPerWarp = DK / kWarps;
  static constexpr int kLoads = kRowsPerWarp / kRowsPerLoad;
  static_assert(DV % 4 == 0 && kLanesPerRow <= 32 && 32 % kLanesPerRow == 0, "dv layout");
  static_assert(DK % kWarps == 0 && kRowsPerWarp % kRowsPerLoad == 0, "dk layout");
};

template <int DK, int DV>
__global__ void __launch_bounds__(256, 2) gdn_decode_kernel(const AveGdnArgs a) {
  using C = DecodeCfg<DK, DV>;
  __shared__ __align__(16) float k_s[DK];
  __shared__ __align__(16) float q_s[DK];
  __shared__ __align__(16) float red[2][C::kWarps][DV];

  const int n = blockIdx.x / a.Hv;
  const int h = blockIdx.x % a.Hv;
  const int hk = h / (a.Hv / a.Hk);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col = (lane % C::kLanesPerRow) * 4;
  const int row0 = warp * C::kRowsPerWarp + lane / C::kLanesPerRow;

  const SeqSpan sp = seq_span(a.cu_seqlens, n, a.T, a.status);
  __nv_bfloat16* o_base = reinterpret_cast<__nv_bfloat16*>(a.o) + sp.b * a.o_stride_b + (int64_t)h * a.o_stride_h;

  int slot = n;
  bool skip = !sp.ok;
  if (a.state_indices != nullptr) {
    slot = a.state_indices[n];
    if (slot >= a.num_slots) {
      if (a.status != nullptr && threadIdx.x == 0) atomicOr(a.status, AVE_GDN_DEV_BAD_SLOT);
      skip = true;
    }
    if (slot < 0) skip = true;
  }
  if (skip) {  // no state access; the sequence's outputs are defined as zero
    for (int t = 0; t < sp.len; ++t)
      if (threadIdx.x < DV) o_base[(int64_t)(sp.t0 + t) * a.o_stride_t + threadIdx.x] = __float2bfloat16(0.f);
    return;
  }

  const int64_t tile = ((int64_t)slot * a.Hv + h) * (int64_t)(DK * DV);
  float4 S[C::kLoads];
  if (a.initial_state != nullptr) {
    const float* src = a.initial_state + tile;
#pragma unroll
    for (int i = 0; i < C::kLoads; ++i)
      S[i] = __ldcs(reinterpret_cast<const float4*>(src + (row0 + i * C::kRowsPerLoad) * DV + col));
  } else {
#pragma unroll
    for (int i = 0; i < C::kLoads; ++i) S[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }

  const __nv_bfloat16* q_base = reinterpret_cast<const __nv_bfloat16*>(a.q) + sp.b * a.q_stride_b + (int64_t)hk * a.q_stride_h;
  const __nv_bfloat16* k_base = reinterpret_cast<const __nv_bfloat16*>(a.k) + sp.b * a.k_stride_b + (int64_t)hk * a.k_stride_h;
  const __nv_bfloat16* v_base = reinterpret_cast<const __nv_bfloat16*>(a.v) + sp.b * a.v_stride_b + (int64_t)h * a.v_stride_h;
  const __nv_bfloat16* z_base = a.z ? reinterpret_cast<const __nv_bfloat16*>(a.z) + sp.b * a.z_stride_b + (int64_t)h * a.z_stride_h : nullptr;
  const float* g_base = a.g + sp.b * a.g_stride_b + h;
  const float* beta_base = a.beta + sp.b * a.g_stride_b + h;
  const bool l2 = (a.flags & AVE_GDN_FLAG_QK_L2NORM) != 0;

  for (int t = 0; t < sp.len; ++t) {
    const int64_t tok = sp.t0 + t;
    if (t > 0) __syncthreads();  // k_s/q_s/red of the previous token are no longer read
    if (threadIdx.x < DK) {
      k_s[threadIdx.x] = bf2f(k_base[tok * a.k_stride_t + threadIdx.x]);
    } else if (threadIdx.x < 2 * DK) {
      q_s[threadIdx.x - DK] = bf2f(q_base[tok * a.q_stride_t + threadIdx.x - DK]);
    }
    float v4[4];
    unpack_bf16x4(*reinterpret_cast<const uint2*>(v_base + tok * a.v_stride_t + col), v4);
    const float alpha = __expf(g_base[tok * a.g_stride_t]);
    const float beta = beta_base[tok * a.g_stride_t];
    __syncthreads();

    // every warp derives k.q and the two norms redundantly from shared memory (no extra barrier)
    float kq = 0.f, kk = 0.f, qq = 0.f;
#pragma unroll
    for (int i = lane; i < DK; i += 32) {
      const float kv = k_s[i], qv = q_s[i];
      kq += kv * qv; kk += kv * kv; qq += qv * qv;
    }
    kq = warp_sum(kq);
    float kn = 1.f, qn = 1.f;
    if (l2) {
      kn = rsqrtf(warp_sum(kk) + 1e-6f);
      qn = rsqrtf(warp_sum(qq) + 1e-6f);
      kq *= kn * qn;
    }

    float r[4] = {0.f, 0.f, 0.f, 0.f}, p[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < C::kLoads; ++i) {
      const int row = row0 + i * C::kRowsPerLoad;
      const float kr = k_s[row] * kn, qr = q_s[row] * qn;
      r[0] += S[i].x * kr; r[1] += S[i].y * kr; r[2] += S[i].z * kr; r[3] += S[i].w * kr;
      p[0] += S[i].x * qr; p[1] += S[i].y * qr; p[2] += S[i].z * qr; p[3] += S[i].w * qr;
    }
    if (C::kRowsPerLoad > 1) {  // lanes that share columns but hold different rows
#pragma unroll
      for (int off = C::kLanesPerRow; off < 32; off <<= 1) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          r[c] += __shfl_xor_sync(0xffffffffu, r[c], off);
          p[c] += __shfl_xor_sync(0xffffffffu, p[c], off);
        }
      }
    }
    if (lane < C::kLanesPerRow) {
      *reinterpret_cast<float4*>(&red[0][warp][col]) = make_float4(r[0], r[1], r[2], r[3]);
      *reinterpret_cast<float4*>(&red[1][warp][col]) = make_float4(p[0], p[1], p[2], p[3]);
    }
    __syncthreads();
    float4 rs = make_float4(0.f, 0.f, 0.f, 0.f), ps = rs;
#pragma unroll
    for (int w = 0; w < C::kWarps; ++w) {
      const float4 x = *reinterpret_cast<const float4*>(&red[0][w][col]);
      const float4 y = *reinterpret_cast<const float4*>(&red[1][w][col]);
      rs.x += x.x; rs.y += x.y; rs.z += x.z; rs.w += x.w;
      ps.x += y.x; ps.y += y.y; ps.z += y.z; ps.w += y.w;
    }
    float u[4], o[4];
    u[0] = beta * (v4[0] - alpha * rs.x); u[1] = beta * (v4[1] - alpha * rs.y);
    u[2] = beta * (v4[2] - alpha * rs.z); u[3] = beta * (v4[3] - alpha * rs.w);
    o[0] = a.scale * (alpha * ps.x + u[0] * kq); o[1] = a.scale * (alpha * ps.y + u[1] * kq);
    o[2] = a.scale * (alpha * ps.z + u[2] * kq); o[3] = a.scale * (alpha * ps.w + u[3] * kq);
#pragma unroll
    for (int i = 0; i < C::kLoads; ++i) {
      const float kr = k_s[row0 + i * C::kRowsPerLoad] * kn;
      S[i].x = alpha * S[i].x + kr * u[0]; S[i].y = alpha * S[i].y + kr * u[1];
      S[i].z = alpha * S[i].z + kr * u[2]; S[i].w = alpha * S[i].w + kr * u[3];
    }
    if (warp == 0) {  // warp 0's first kLanesPerRow lanes cover every column once
      if (z_base != nullptr) {
        float zz[4];
        unpack_bf16x4(*reinterpret_cast<const uint2*>(z_base + tok * a.z_stride_t + col), zz);
        const bool gate_first = (a.flags & AVE_GDN_FLAG_GATE_FIRST) != 0;
        if (gate_first) {
#pragma unroll
          for (int c = 0; c < 4; ++c) o[c] *= silu(zz[c]);
        }
        float ss = o[0] * o[0] + o[1] * o[1] + o[2] * o[2] + o[3] * o[3];
        if (lane >= C::kLanesPerRow) ss = 0.f;
        ss = warp_sum(ss);
        const float rinv = rsqrtf(ss * (1.0f / DV) + a.norm_eps);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const float w = a.norm_weight ? a.norm_weight[col + c] : 1.0f;
          o[c] = o[c] * rinv * w * (gate_first ? 1.0f : silu(zz[c]));
        }
      }
      if (lane < C::kLanesPerRow) {
        uint2 packed = make_uint2(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]));
        *reinterpret_cast<uint2*>(o_base + tok * a.o_stride_t + col) = packed;
      }
    }
  }

  if (a.final_state != nullptr) {
    float* dst = a.final_state + tile;
#pragma unroll
    for (int i = 0; i < C::kLoads; ++i)
      __stcs(reinterpret_cast<float4*>(dst + (row0 + i * C::kRowsPerLoad) * DV + col), S[i]);
  }
}

// Single-token step over a slot pool (T == 1), persistent form: each CTA walks tiles blockIdx.x, +gridDim.x, ...
// While one 64 KiB tile is being reduced, updated and streamed out of registers, the next one is already landing
// in shared memory through one bulk copy, so loads stay in flight across the compute and store phases.
__global__ void __launch_bounds__(256, 2) gdn_decode_pool_kernel(const AveGdnArgs a, int n_tiles) {
  constexpr int DK = 128, DV = 128;
  using C = DecodeCfg<DK, DV>;
  extern __shared__ __align__(128) uint8_t dyn_smem[];
  float* tile_s = reinterpret_cast<float*>(dyn_smem);  // [DK][DV] fp32
  __shared__ __align__(16) float k_s[DK];
  __shared__ __align__(16) float q_s[DK];
  __shared__ __align__(16) float red[2][C::kWarps][DV];
  __shared__ uint64_t full_bar;
  __shared__ uint32_t abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col = lane * 4;
  const int row0 = warp * C::kRowsPerWarp;
  const bool l2 = (a.flags & AVE_GDN_FLAG_QK_L2NORM) != 0;

  auto slot_of = [&](int t) -> int {  // < 0: the tile is skipped
    const int n = t / a.Hv;
    int slot = a.state_indices ? a.state_indices[n] : n;
    if (slot >= a.num_slots) {
      if (a.status != nullptr && threadIdx.x == 0) atomicOr(a.status, AVE_GDN_DEV_BAD_SLOT);
      slot = -1;
    }
    return slot;
  };
  auto tile_offset = [&](int t, int slot) -> int64_t { return ((int64_t)slot * a.Hv + (t % a.Hv)) * (int64_t)(DK * DV); };

  int t = blockIdx.x;
  if (t >= n_tiles) return;
  int slot = slot_of(t);
  if (threadIdx.x == 0) {
    tc::mbar_init(&full_bar, 1);
    abort_flag = 0;
    tc::fence_barrier_init();
    if (slot >= 0) {
      tc::mbar_expect_tx(&full_bar, DK * DV * 4);
      tc::bulk_load(tile_s, a.initial_state + tile_offset(t, slot), DK * DV * 4, &full_bar);
    }
  }
  __syncthreads();
  uint32_t phase = 0;

  // per-token inputs (one k or q element per thread, four v elements, gate and beta) are fetched one tile ahead
  struct Small { float kq_elem; uint2 v; float g, beta; };
  auto fetch_small = [&](int tt) -> Small {
    Small sm;
    const int n = tt / a.Hv, h = tt % a.Hv, hk = h / (a.Hv / a.Hk);
    const __nv_bfloat16* src = (threadIdx.x < DK)
        ? reinterpret_cast<const __nv_bfloat16*>(a.k) + n * a.k_stride_b + (int64_t)hk * a.k_stride_h + threadIdx.x
        : reinterpret_cast<const __nv_bfloat16*>(a.q) + n * a.q_stride_b + (int64_t)hk * a.q_stride_h + (threadIdx.x - DK);
    sm.kq_elem = bf2f(*src);
    sm.v = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(a.v) + n * a.v_stride_b + (int64_t)h * a.v_stride_h + col);
    sm.g = a.g[n * a.g_stride_b + h];
    sm.beta = a.beta[n * a.g_stride_b + h];
    return sm;
  };
  Small cur = fetch_small(t);

  for (; t < n_tiles; t += gridDim.x) {
    const int n = t / a.Hv, h = t % a.Hv;
    const int t_next = t + gridDim.x;
    const int slot_next = (t_next < n_tiles) ? slot_of(t_next) : -1;
    Small nxt = cur;
    if (t_next < n_tiles) nxt = fetch_small(t_next);
    __nv_bfloat16* o_ptr = reinterpret_cast<__nv_bfloat16*>(a.o) + n * a.o_stride_b + (int64_t)h * a.o_stride_h;

    float4 S[C::kLoads];
    bool ok = true;
    if (slot >= 0) {
      ok = tc::mbar_wait(&full_bar, phase, &abort_flag);
      phase ^= 1u;
#pragma unroll
      for (int i = 0; i < C::kLoads; ++i) S[i] = *reinterpret_cast<const float4*>(tile_s + (row0 + i) * DV + col);
    }
    // every thread has its part of the tile in registers (and is done with k_s/q_s/red of the previous tile)
    if (__syncthreads_or(!ok)) {
      if (threadIdx.x == 0 && a.status != nullptr) atomicOr(a.status, AVE_GDN_DEV_WAIT_EXPIRED);
      return;
    }
    if (threadIdx.x == 0 && slot_next >= 0) {
      tc::mbar_expect_tx(&full_bar, DK * DV * 4);
      tc::bulk_load(tile_s, a.initial_state + tile_offset(t_next, slot_next), DK * DV * 4, &full_bar);
    }
    if (slot < 0) {
      if (threadIdx.x < DV) o_ptr[threadIdx.x] = __float2bfloat16(0.f);
      slot = slot_next;
      cur = nxt;
      continue;
    }
    if (threadIdx.x < DK) k_s[threadIdx.x] = cur.kq_elem;
    else q_s[threadIdx.x - DK] = cur.kq_elem;
    float v4[4];
    unpack_bf16x4(cur.v, v4);
    const float alpha = __expf(cur.g);
    const float beta = cur.beta;
    __syncthreads();

    float kq = 0.f, kk = 0.f, qq = 0.f;
#pragma unroll
    for (int i = lane; i < DK; i += 32) {
      const float kv = k_s[i], qv = q_s[i];
      kq += kv * qv; kk += kv * kv; qq += qv * qv;
    }
    kq = warp_sum(kq);
    float kn = 1.f, qn = 1.f;
    if (l2) {
      kn = rsqrtf(warp_sum(kk) + 1e-6f);
      qn = rsqrtf(warp_sum(qq) + 1e-6f);
      kq *= kn * qn;
    }
    float r[4] = {0.f, 0.f, 0.f, 0.f}, p[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < C::kLoads; ++i) {
      const float kr = k_s[row0 + i] * kn, qr = q_s[row0 + i] * qn;
      r[0] += S[i].x * kr; r[1] += S[i].y * kr; r[2] += S[i].z * kr; r[3] += S[i].w * kr;
      p[0] += S[i].x * qr; p[1] += S[i].y * qr; p[2] += S[i].z * qr; p[3] += S[i].w * qr;
    }
    *reinterpret_cast<float4*>(&red[0][warp][col]) = make_float4(r[0], r[1], r[2], r[3]);
    *reinterpret_cast<float4*>(&red[1][warp][col]) = make_float4(p[0], p[1], p[2], p[3]);
    __syncthreads();
    float4 rs = make_float4(0.f, 0.f, 0.f, 0.f), ps = rs;
#pragma unroll
    for (int w = 0; w < C::kWarps; ++w) {
      const float4 x = *reinterpret_cast<const float4*>(&red[0][w][col]);
      const float4 y = *reinterpret_cast<const float4*>(&red[1][w][col]);
      rs.x += x.x; rs.y += x.y; rs.z += x.z; rs.w += x.w;
      ps.x += y.x; ps.y += y.y; ps.z += y.z; ps.w += y.w;
    }
    float u[4], o[4];
    u[0] = beta * (v4[0] - alpha * rs.x); u[1] = beta * (v4[1] - alpha * rs.y);
    u[2] = beta * (v4[2] - alpha * rs.z); u[3] = beta * (v4[3] - alpha * rs.w);
    o[0] = a.scale * (alpha * ps.x + u[0] * kq); o[1] = a.scale * (alpha * ps.y + u[1] * kq);
    o[2] = a.scale * (alpha * ps.z + u[2] * kq); o[3] = a.scale * (alpha * ps.w + u[3] * kq);
    float* dst = a.final_state + tile_offset(t, slot);
#pragma unroll
    for (int i = 0; i < C::kLoads; ++i) {
      const float kr = k_s[row0 + i] * kn;
      S[i].x = alpha * S[i].x + kr * u[0]; S[i].y = alpha * S[i].y + kr * u[1];
      S[i].z = alpha * S[i].z + kr * u[2]; S[i].w = alpha * S[i].w + kr * u[3];
      __stcs(reinterpret_cast<float4*>(dst + (row0 + i) * DV + col), S[i]);
    }
    if (warp == 0) {
      if (a.z != nullptr) {
        float zz[4];
        unpack_bf16x4(*reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(a.z) + n * a.z_stride_b +
                                                      (int64_t)h * a.z_stride_h + col), zz);
        const bool gate_first = (a.flags & AVE_GDN_FLAG_GATE_FIRST) != 0;
        if (gate_first) {
#pragma unroll
          for (int c = 0; c < 4; ++c) o[c] *= silu(zz[c]);
        }
        const float ss = warp_sum(o[0] * o[0] + o[1] * o[1] + o[2] * o[2] + o[3] * o[3]);
        const float rinv = rsqrtf(ss * (1.0f / DV) + a.norm_eps);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const float w = a.norm_weight ? a.norm_weight[col + c] : 1.0f;
          o[c] = o[c] * rinv * w * (gate_first ? 1.0f : silu(zz[c]));
        }
      }
      *reinterpret_cast<uint2*>(o_ptr + col) = make_uint2(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]));
    }
    slot = slot_next;
    cur = nxt;
  }
}

int launch_decode(const AveGdnArgs& a, cudaStream_t stream) {
  const unsigned grid = (unsigned)a.n_seqs * (unsigned)a.Hv;
  if (grid == 0) return AVE_GDN_OK;
  // one token per sequence over an existing pool that is updated in place or written elsewhere: persistent form
  if (a.dk == 128 && a.dv == 128 && a.T == 1 && a.cu_seqlens == nullptr && a.initial_state != nullptr && a.final_state != nullptr) {
    static bool attr_set_dev[64] = {};
    int dev = 0, sms = 148;
    AVE_CUDA_TRY(cudaGetDevice(&dev));
    if (!attr_set_dev[dev & 63]) {
      AVE_CUDA_TRY(cudaFuncSetAttribute(gdn_decode_pool_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 128 * 4));
      attr_set_dev[dev & 63] = true;
    }
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const unsigned persistent = (unsigned)(2 * sms);
    gdn_decode_pool_kernel<<<grid < persistent ? grid : persistent, 256, 128 * 128 * 4, stream>>>(a, (int)grid);
  } else if (a.dk == 128 && a.dv == 128) {
    gdn_decode_kernel<128, 128><<<grid, 256, 0, stream>>>(a);
  } else if (a.dk == 64 && a.dv == 64) {
    gdn_decode_kernel<64, 64><<<grid, 256, 0, stream>>>(a);
  } else {
    return AVE_GDN_UNSUPPORTED;
  }
  AVE_CUDA_TRY(cudaGetLastError());
  return AVE_GDN_OK;
}

}  // namespace ave
