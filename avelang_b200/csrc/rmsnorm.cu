// Gated RMSNorm over rows of d = 64 or 128 elements:  y = w * x * rsqrt(mean(x^2) + eps) * silu(z).
// Pure streaming: one half-warp per row, 16-byte (d=128) or 8-byte (d=64) bf16 loads per lane, fp32 math.
#include "common.cuh"

namespace ave {

// Rows are indexed (batch, token, head); a launch covers `batches` batch rows of rows_per_batch = tokens * heads rows
// each (the public entry point passes one batch).
struct NormBatch {
  int64_t rows_per_batch;
  int64_t xs_b, zs_b, ys_b;
};

// D = 128: a half-warp per row, eight elements (16 bytes of bf16, 32 of fp32) per lane, two rows in flight per
// half-warp; D = 64: same with four elements per lane.  Rows are (batch, token, head) in that order.  Like the other
// streaming helpers the kernel is bound by instruction issue before HBM, so the math runs on packed fp32 pairs and
// tensors whose rows are evenly spaced (`flat`) skip the per-row index divisions.
template <int D, typename XT>
__global__ void __launch_bounds__(256) gated_rmsnorm_kernel(const XT* __restrict__ x, const __nv_bfloat16* __restrict__ z,
                                                            const float* __restrict__ w, __nv_bfloat16* __restrict__ y,
                                                            int64_t rows, int heads, int64_t xs_t, int64_t xs_h,
                                                            int64_t zs_t, int64_t zs_h, int64_t ys_t, int64_t ys_h,
                                                            float eps, int gate_first, const void* const* __restrict__ peers,
                                                            int n_peers, int64_t peer_off, NormBatch nb, int flat) {
  constexpr int E = D / 16;  // elements per lane: 8 or 4
  constexpr int P = E / 2;   // pairs per lane
  constexpr int U = 2;       // rows in flight per half-warp
  const int sub = threadIdx.x & 15;  // lane inside the half-warp
  const int64_t hw_global = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 4;
  const int64_t n_hw = ((int64_t)gridDim.x * blockDim.x) >> 4;
  float2 wv[P];
#pragma unroll
  for (int i = 0; i < P; ++i) wv[i] = w ? make_float2(w[sub * E + 2 * i], w[sub * E + 2 * i + 1]) : make_float2(1.f, 1.f);
  for (int64_t r0 = hw_global; r0 < rows; r0 += U * n_hw) {
    float2 xv[U][P], zv[U][P];
    int64_t yoff[U];
    bool live[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t r = r0 + u * n_hw;
      live[u] = r < rows;
      if (!live[u]) {
#pragma unroll
        for (int i = 0; i < P; ++i) { xv[u][i] = make_float2(0.f, 0.f); zv[u][i] = make_float2(0.f, 0.f); }
        yoff[u] = 0;
        continue;
      }
      int64_t xo, zo;
      if (flat) {  // row r sits r head-strides from the base in all three tensors
        xo = r * xs_h; zo = r * zs_h; yoff[u] = r * ys_h + sub * E;
      } else {
        // 32-bit index arithmetic (the launcher checks the row count): 64-bit divisions would dominate this kernel
        const uint32_t r32 = (uint32_t)r, rpb = (uint32_t)nb.rows_per_batch;
        const uint32_t b = r32 / rpb, rr = r32 - b * rpb;
        const uint32_t t = rr / (uint32_t)heads;
        const int h = (int)(rr - t * (uint32_t)heads);
        xo = (int64_t)b * nb.xs_b + (int64_t)t * xs_t + h * xs_h;
        zo = (int64_t)b * nb.zs_b + (int64_t)t * zs_t + h * zs_h;
        yoff[u] = (int64_t)b * nb.ys_b + (int64_t)t * ys_t + h * ys_h + sub * E;
      }
      const XT* xr = x + xo + sub * E;
      const __nv_bfloat16* zr = z + zo + sub * E;
      if constexpr (sizeof(XT) == 4) {
#pragma unroll
        for (int i = 0; i < P; i += 2) {
          const float4 v4 = *reinterpret_cast<const float4*>(xr + 2 * i);
          xv[u][i] = make_float2(v4.x, v4.y); xv[u][i + 1] = make_float2(v4.z, v4.w);
        }
      } else if constexpr (E == 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(xr);
        xv[u][0] = bf16x2_to_float2(raw.x); xv[u][1] = bf16x2_to_float2(raw.y);
        xv[u][2] = bf16x2_to_float2(raw.z); xv[u][3] = bf16x2_to_float2(raw.w);
      } else {
        const uint2 raw = *reinterpret_cast<const uint2*>(xr);
        xv[u][0] = bf16x2_to_float2(raw.x); xv[u][1] = bf16x2_to_float2(raw.y);
      }
      if constexpr (E == 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(zr);
        zv[u][0] = bf16x2_to_float2(raw.x); zv[u][1] = bf16x2_to_float2(raw.y);
        zv[u][2] = bf16x2_to_float2(raw.z); zv[u][3] = bf16x2_to_float2(raw.w);
      } else {
        const uint2 raw = *reinterpret_cast<const uint2*>(zr);
        zv[u][0] = bf16x2_to_float2(raw.x); zv[u][1] = bf16x2_to_float2(raw.y);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float2 ss2 = make_float2(0.f, 0.f);
#pragma unroll
      for (int i = 0; i < P; ++i) {
        zv[u][i] = silu2(zv[u][i]);
        if (gate_first) xv[u][i] = __fmul2_rn(xv[u][i], zv[u][i]);
        ss2 = __ffma2_rn(xv[u][i], xv[u][i], ss2);
      }
      float ss = ss2.x + ss2.y;
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);  // stays inside the half-warp
      const float rinv = rsqrtf(ss * (1.0f / D) + eps);
      uint32_t packed[P];
#pragma unroll
      for (int i = 0; i < P; ++i) {
        float2 o2 = __fmul2_rn(__fmul2_rn(xv[u][i], make_float2(rinv, rinv)), wv[i]);
        if (!gate_first) o2 = __fmul2_rn(o2, zv[u][i]);
        packed[i] = pack_bf16x2(o2.x, o2.y);
      }
      if (!live[u]) continue;
      if (n_peers > 0) {  // fused all-gather: the same row goes to every GPU's buffer (plain peer stores)
        for (int p = 0; p < n_peers; ++p) {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(peers[p])) + peer_off + yoff[u];
          if constexpr (E == 8) *reinterpret_cast<uint4*>(dst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
          else *reinterpret_cast<uint2*>(dst) = make_uint2(packed[0], packed[1]);
        }
      } else {
        if constexpr (E == 8) *reinterpret_cast<uint4*>(y + yoff[u]) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        else *reinterpret_cast<uint2*>(y + yoff[u]) = make_uint2(packed[0], packed[1]);
      }
    }
  }
}

template <typename XT>
static int launch_norm_t(const XT* x, const AveGdnNormArgs& a, cudaStream_t stream, const void* const* peers = nullptr, int n_peers = 0,
                         int64_t peer_off = 0, int batches = 1, int64_t xs_b = 0, int64_t zs_b = 0, int64_t ys_b = 0) {
  if (a.rows == 0 || batches == 0) return AVE_GDN_OK;
  const NormBatch nb{a.rows, xs_b, zs_b, ys_b};
  const int64_t rows = a.rows * batches;
  if (rows >= ((int64_t)1 << 31) || a.heads <= 0) return AVE_GDN_UNSUPPORTED;
  const int64_t blocks_needed = (rows + 31) / 32;  // 16 half-warps per block, two rows per half-warp and pass
  const unsigned grid = (unsigned)(blocks_needed < 148 * 64 ? blocks_needed : 148 * 64);
  const int gate_first = (a.flags & AVE_GDN_FLAG_GATE_FIRST) ? 1 : 0;
  // evenly spaced rows: token stride = heads x head stride in every tensor, and batch rows follow one another the same way
  const bool even = a.x_stride_t == a.heads * a.x_stride_h && a.z_stride_t == a.heads * a.z_stride_h && a.y_stride_t == a.heads * a.y_stride_h;
  const int flat = (even && (batches == 1 || (xs_b == a.rows * a.x_stride_h && zs_b == a.rows * a.z_stride_h && ys_b == a.rows * a.y_stride_h))) ? 1 : 0;
  const __nv_bfloat16* z = reinterpret_cast<const __nv_bfloat16*>(a.z);
  __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(a.y);
  if (a.d == 128) {
    gated_rmsnorm_kernel<128, XT><<<grid, 256, 0, stream>>>(x, z, a.weight, y, rows, a.heads, a.x_stride_t, a.x_stride_h,
                                                            a.z_stride_t, a.z_stride_h, a.y_stride_t, a.y_stride_h, a.eps, gate_first, peers, n_peers, peer_off, nb, flat);
  } else if (a.d == 64) {
    gated_rmsnorm_kernel<64, XT><<<grid, 256, 0, stream>>>(x, z, a.weight, y, rows, a.heads, a.x_stride_t, a.x_stride_h,
                                                           a.z_stride_t, a.z_stride_h, a.y_stride_t, a.y_stride_h, a.eps, gate_first, nullptr, 0, 0, nb, flat);
  } else {
    return AVE_GDN_UNSUPPORTED;
  }
  AVE_CUDA_TRY(cudaGetLastError());
  return AVE_GDN_OK;
}

int launch_gated_rmsnorm(const AveGdnNormArgs& a, cudaStream_t stream) {
  return launch_norm_t(reinterpret_cast<const __nv_bfloat16*>(a.x), a, stream);
}

// fp32 input variant used by the prefill path when the un-normalised output is staged in scratch
int launch_gated_rmsnorm_f32in(const AveGdnNormArgs& a, cudaStream_t stream, const void* const* peers, int n_peers, int64_t peer_off) {
  return launch_norm_t(reinterpret_cast<const float*>(a.x), a, stream, peers, n_peers, peer_off);
}

// The same over `batches` batch rows in one launch: a.rows counts the rows of one batch row, the strides step between them.
int launch_gated_rmsnorm_f32in_batched(const AveGdnNormArgs& a, cudaStream_t stream, const void* const* peers, int n_peers,
                                       int64_t peer_off, int batches, int64_t xs_b, int64_t zs_b, int64_t ys_b) {
  return launch_norm_t(reinterpret_cast<const float*>(a.x), a, stream, peers, n_peers, peer_off, batches, xs_b, zs_b, ys_b);
}

}  // namespace ave
