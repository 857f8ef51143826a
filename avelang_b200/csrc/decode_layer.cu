// One decode step of a whole gated-delta-net layer behind its in-projection, as ONE kernel: per sequence the new
// token's projection row [q | k | v | z | b | a] goes through
//   causal conv1d update (+ SiLU) on the q, k, v channels, history shifted in place in its slot pool
//   -> L2 norm of q and k per head -> g = -exp(A_log) softplus(a + dt_bias), beta = sigmoid(b)
//   -> the gated-delta-rule update of the fp32 state tile in its slot (streamed once in, once out)
//   -> gated RMSNorm with z
// so that a decode layer is two launches (the projection GEMM and this kernel) instead of five.  The state streaming
// is that of the slot-pool decode kernel: persistent CTAs, the next 64 KiB tile lands in shared memory through a bulk
// copy while the current one is reduced, updated and streamed out of registers.  A CTA takes a (sequence, key head) at
// a time and walks the value heads that share it back to back: q and k are convolved and their history shifted once,
// by the one CTA that reads them, which is what makes the in-place history update free of races.
// Rounding points are those of the separate kernels (convolution outputs are rounded to bf16, g and beta stay fp32), so
// the fused step leaves the states and histories that conv1d_update + gate_beta + decode_step leave, bit for bit.
#include "common.cuh"
#include "tc.cuh"

namespace ave {
namespace {

constexpr int DK = 128, DV = 128, WARPS = 8, ROWS = DK / WARPS;  // rows of the tile per warp; a lane owns 4 columns

template <int WIDTH>
__global__ void __launch_bounds__(256, 2) gdn_decode_layer_kernel(const AveGdnDecodeLayerArgs a, int n_units) {
  extern __shared__ __align__(128) uint8_t dyn_smem[];
  float* tile_s = reinterpret_cast<float*>(dyn_smem);  // [DK][DV] fp32
  __shared__ __align__(16) float k_s[DK];
  __shared__ __align__(16) float q_s[DK];
  __shared__ __align__(16) float v_s[DV];
  __shared__ __align__(16) float red[2][WARPS][DV];
  __shared__ uint64_t full_bar;
  __shared__ uint32_t abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int col = lane * 4, row0 = warp * ROWS;
  const int r = a.Hv / a.Hk;                    // value heads per key head
  const int Cn = 2 * a.Hk * DK + a.Hv * DV;     // convolved channels: q | k | v
  const int off_k = a.Hk * DK, off_v = 2 * a.Hk * DK, off_z = off_v + a.Hv * DV, off_b = off_z + a.Hv * DV, off_a = off_b + a.Hv;
  const __nv_bfloat16* proj = reinterpret_cast<const __nv_bfloat16*>(a.proj);
  const __nv_bfloat16* cw = reinterpret_cast<const __nv_bfloat16*>(a.conv_w);
  const __nv_bfloat16* cb = reinterpret_cast<const __nv_bfloat16*>(a.conv_bias);
  __nv_bfloat16* cstate = reinterpret_cast<__nv_bfloat16*>(a.conv_state);

  if ((int)blockIdx.x >= n_units) return;
  const int n_local = ((n_units - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x) * r;  // tiles this CTA walks
  auto unit_of = [&](int i) { return (int)blockIdx.x + (i / r) * (int)gridDim.x; };
  auto slot_of_seq = [&](int n) -> int {  // < 0: the sequence is skipped
    int slot = a.state_indices ? a.state_indices[n] : n;
    if (slot >= a.num_slots) {
      if (a.status != nullptr && tid == 0) atomicOr(a.status, AVE_GDN_DEV_BAD_SLOT);
      slot = -1;
    }
    return slot;
  };
  auto tile_ptr = [&](int slot, int h) { return a.state_pool + ((int64_t)slot * a.Hv + h) * (int64_t)(DK * DV); };
  // one channel of the convolution for sequence n: history of slot `slot` plus the new input; the history is shifted
  // in place by this (the only) thread that reads the channel.  Same arithmetic order as the standalone update kernel.
  auto conv_channel = [&](int n, int slot, int ch) -> float {
    __nv_bfloat16* st = cstate + (int64_t)slot * (WIDTH - 1) * Cn + ch;
    __nv_bfloat16 x[WIDTH];
#pragma unroll
    for (int j = 0; j < WIDTH - 1; ++j) x[j] = st[(int64_t)j * Cn];
    x[WIDTH - 1] = proj[(int64_t)n * a.proj_stride + ch];
    float acc = cb ? bf2f(cb[ch]) : 0.f;
#pragma unroll
    for (int j = 0; j < WIDTH; ++j) acc = fmaf(bf2f(cw[(int64_t)ch * WIDTH + j]), bf2f(x[j]), acc);
#pragma unroll
    for (int j = 0; j < WIDTH - 1; ++j) st[(int64_t)j * Cn] = x[j + 1];
    return bf2f(__float2bfloat16(silu(acc)));  // the separate kernels store the convolution output as bf16
  };

  int slot = slot_of_seq(unit_of(0) / a.Hk);
  if (tid == 0) {
    tc::mbar_init(&full_bar, 1);
    abort_flag = 0;
    tc::fence_barrier_init();
    if (slot >= 0) {
      tc::mbar_expect_tx(&full_bar, DK * DV * 4);
      tc::bulk_load(tile_s, tile_ptr(slot, (unit_of(0) % a.Hk) * r), DK * DV * 4, &full_bar);
    }
  }
  __syncthreads();
  uint32_t phase = 0;

  for (int i = 0; i < n_local; ++i) {
    const int u = unit_of(i), n = u / a.Hk, hk = u % a.Hk, j = i % r, h = hk * r + j;
    int slot_next = -1, h_next = 0;
    if (i + 1 < n_local) {
      const int u2 = unit_of(i + 1);
      slot_next = (u2 == u) ? slot : slot_of_seq(u2 / a.Hk);
      h_next = (u2 % a.Hk) * r + (i + 1) % r;
    }
    __nv_bfloat16* o_ptr = reinterpret_cast<__nv_bfloat16*>(a.o) + (int64_t)n * a.o_stride + h * DV;

    // this token's small inputs, computed while the tile is still landing
    float kq_elem = 0.f, v_elem = 0.f, g = 0.f, beta = 0.f;
    if (slot >= 0) {
      if (j == 0) kq_elem = conv_channel(n, slot, tid < DK ? off_k + hk * DK + tid : hk * DK + (tid - DK));
      if (tid < DV) v_elem = conv_channel(n, slot, off_v + h * DV + tid);
      const float av = bf2f(proj[(int64_t)n * a.proj_stride + off_a + h]) + a.dt_bias[h];
      const float bv = bf2f(proj[(int64_t)n * a.proj_stride + off_b + h]);
      const float sp = av > 20.f ? av : log1pf(expf(av));  // softplus
      g = -expf(a.A_log[h]) * sp;
      beta = 1.0f / (1.0f + expf(-bv));
    }

    float4 S[ROWS];
    bool ok = true;
    if (slot >= 0) {
      ok = tc::mbar_wait(&full_bar, phase, &abort_flag);
      phase ^= 1u;
#pragma unroll
      for (int rr = 0; rr < ROWS; ++rr) S[rr] = *reinterpret_cast<const float4*>(tile_s + (row0 + rr) * DV + col);
    }
    // every thread has its part of the tile in registers (and is done with the shared vectors of the previous tile)
    if (__syncthreads_or(!ok)) {
      if (tid == 0 && a.status != nullptr) atomicOr(a.status, AVE_GDN_DEV_WAIT_EXPIRED);
      return;
    }
    if (tid == 0 && slot_next >= 0) {
      tc::mbar_expect_tx(&full_bar, DK * DV * 4);
      tc::bulk_load(tile_s, tile_ptr(slot_next, h_next), DK * DV * 4, &full_bar);
    }
    if (slot < 0) {
      if (tid < DV) o_ptr[tid] = __float2bfloat16(0.f);
      slot = slot_next;
      continue;
    }
    if (j == 0) {
      if (tid < DK) k_s[tid] = kq_elem;
      else q_s[tid - DK] = kq_elem;
    }
    if (tid < DV) v_s[tid] = v_elem;
    const float alpha = __expf(g);
    __syncthreads();

    const float4 vv = *reinterpret_cast<const float4*>(v_s + col);
    const float v4[4] = {vv.x, vv.y, vv.z, vv.w};
    float kq = 0.f, kk = 0.f, qq = 0.f;
#pragma unroll
    for (int e = lane; e < DK; e += 32) {
      const float kv = k_s[e], qv = q_s[e];
      kq += kv * qv; kk += kv * kv; qq += qv * qv;
    }
    kq = warp_sum(kq);
    const float kn = rsqrtf(warp_sum(kk) + 1e-6f), qn = rsqrtf(warp_sum(qq) + 1e-6f);
    kq *= kn * qn;
    float rsum[4] = {0.f, 0.f, 0.f, 0.f}, psum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int rr = 0; rr < ROWS; ++rr) {
      const float kr = k_s[row0 + rr] * kn, qr = q_s[row0 + rr] * qn;
      rsum[0] += S[rr].x * kr; rsum[1] += S[rr].y * kr; rsum[2] += S[rr].z * kr; rsum[3] += S[rr].w * kr;
      psum[0] += S[rr].x * qr; psum[1] += S[rr].y * qr; psum[2] += S[rr].z * qr; psum[3] += S[rr].w * qr;
    }
    *reinterpret_cast<float4*>(&red[0][warp][col]) = make_float4(rsum[0], rsum[1], rsum[2], rsum[3]);
    *reinterpret_cast<float4*>(&red[1][warp][col]) = make_float4(psum[0], psum[1], psum[2], psum[3]);
    __syncthreads();
    float4 rs = make_float4(0.f, 0.f, 0.f, 0.f), ps = rs;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float4 x = *reinterpret_cast<const float4*>(&red[0][w][col]);
      const float4 y = *reinterpret_cast<const float4*>(&red[1][w][col]);
      rs.x += x.x; rs.y += x.y; rs.z += x.z; rs.w += x.w;
      ps.x += y.x; ps.y += y.y; ps.z += y.z; ps.w += y.w;
    }
    float uu[4], o[4];
    uu[0] = beta * (v4[0] - alpha * rs.x); uu[1] = beta * (v4[1] - alpha * rs.y);
    uu[2] = beta * (v4[2] - alpha * rs.z); uu[3] = beta * (v4[3] - alpha * rs.w);
    o[0] = a.scale * (alpha * ps.x + uu[0] * kq); o[1] = a.scale * (alpha * ps.y + uu[1] * kq);
    o[2] = a.scale * (alpha * ps.z + uu[2] * kq); o[3] = a.scale * (alpha * ps.w + uu[3] * kq);
    float* dst = tile_ptr(slot, h);
#pragma unroll
    for (int rr = 0; rr < ROWS; ++rr) {
      const float kr = k_s[row0 + rr] * kn;
      S[rr].x = alpha * S[rr].x + kr * uu[0]; S[rr].y = alpha * S[rr].y + kr * uu[1];
      S[rr].z = alpha * S[rr].z + kr * uu[2]; S[rr].w = alpha * S[rr].w + kr * uu[3];
      __stcs(reinterpret_cast<float4*>(dst + (row0 + rr) * DV + col), S[rr]);
    }
    if (warp == 0) {  // gated RMSNorm with this head's z columns of the projection row
      float zz[4];
      unpack_bf16x4(*reinterpret_cast<const uint2*>(proj + (int64_t)n * a.proj_stride + off_z + h * DV + col), zz);
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
      *reinterpret_cast<uint2*>(o_ptr + col) = make_uint2(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]));
    }
    slot = slot_next;
  }
}

}  // namespace

int launch_decode_layer(const AveGdnDecodeLayerArgs& a, cudaStream_t stream) {
  const int units = a.n_seqs * a.Hk;
  if (units == 0) return AVE_GDN_OK;
  static bool attr_set_dev[64] = {};
  int dev = 0, sms = 148;
  AVE_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return AVE_GDN_UNSUPPORTED;
  if (!attr_set_dev[dev]) {
    AVE_CUDA_TRY(cudaFuncSetAttribute(gdn_decode_layer_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, DK * DV * 4));
    AVE_CUDA_TRY(cudaFuncSetAttribute(gdn_decode_layer_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, DK * DV * 4));
    AVE_CUDA_TRY(cudaFuncSetAttribute(gdn_decode_layer_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, DK * DV * 4));
    attr_set_dev[dev] = true;  // repeating the three calls from another thread is harmless
  }
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const unsigned grid = (unsigned)(units < 2 * sms ? units : 2 * sms);
  switch (a.width) {
    case 2: gdn_decode_layer_kernel<2><<<grid, 256, DK * DV * 4, stream>>>(a, units); break;
    case 3: gdn_decode_layer_kernel<3><<<grid, 256, DK * DV * 4, stream>>>(a, units); break;
    case 4: gdn_decode_layer_kernel<4><<<grid, 256, DK * DV * 4, stream>>>(a, units); break;
    default: return AVE_GDN_UNSUPPORTED;
  }
  AVE_CUDA_TRY(cudaGetLastError());
  return AVE_GDN_OK;
}

}  // namespace ave
