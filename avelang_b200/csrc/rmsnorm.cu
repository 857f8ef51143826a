// Gated RMSNorm over rows of d = 64 or 128 elements:  y = w * x * rsqrt(mean(x^2) + eps) * silu(z).
// Pure streaming: one warp per row, 8-byte (d=128) or 4-byte (d=64) loads per lane, fp32 math.
#include "common.cuh"

namespace ave {

// Rows are indexed (batch, token, head); a launch covers `batches` batch rows of rows_per_batch = tokens * heads rows
// each (the public entry point passes one batch).
struct NormBatch {
  int64_t rows_per_batch;
  int64_t xs_b, zs_b, ys_b;
};

template <int D, typename XT>
__global__ void __launch_bounds__(256) gated_rmsnorm_kernel(const XT* __restrict__ x, const __nv_bfloat16* __restrict__ z,
                                                            const float* __restrict__ w, __nv_bfloat16* __restrict__ y,
                                                            int64_t rows, int heads, int64_t xs_t, int64_t xs_h,
                                                            int64_t zs_t, int64_t zs_h, int64_t ys_t, int64_t ys_h,
                                                            float eps, int gate_first, const void* const* __restrict__ peers,
                                                            int n_peers, int64_t peer_off, NormBatch nb) {
  constexpr int E = D / 32;  // elements per lane
  constexpr int U = 1;       // rows in flight per warp (2 and 4 were measured: 4 % and 12 % slower on 786 k rows)
  const int lane = threadIdx.x & 31;
  const int64_t warp_global = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t n_warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t r0 = warp_global; r0 < rows; r0 += U * n_warps) {
    float xv[U][E], zv[U][E];
    int64_t yoff[U];
    bool live[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t r = r0 + u * n_warps;
      live[u] = r < rows;
      if (!live[u]) continue;
      // 32-bit index arithmetic (the launcher checks the row count): 64-bit divisions would dominate this kernel
      const uint32_t r32 = (uint32_t)r, rpb = (uint32_t)nb.rows_per_batch;
      const uint32_t b = r32 / rpb, rr = r32 - b * rpb;
      const uint32_t t = rr / (uint32_t)heads;
      const int h = (int)(rr - t * (uint32_t)heads);
      const XT* xr = x + (int64_t)b * nb.xs_b + (int64_t)t * xs_t + h * xs_h + lane * E;
      const __nv_bfloat16* zr = z + (int64_t)b * nb.zs_b + (int64_t)t * zs_t + h * zs_h + lane * E;
      yoff[u] = (int64_t)b * nb.ys_b + (int64_t)t * ys_t + h * ys_h + lane * E;
      if constexpr (sizeof(XT) == 4 && E == 4) {
        const float4 v4 = *reinterpret_cast<const float4*>(xr);
        xv[u][0] = v4.x; xv[u][1] = v4.y; xv[u][2] = v4.z; xv[u][3] = v4.w;
      } else if constexpr (sizeof(XT) == 4) {
        const float2 v2 = *reinterpret_cast<const float2*>(xr);
        xv[u][0] = v2.x; xv[u][1] = v2.y;
      } else if constexpr (E == 4) {
        unpack_bf16x4(*reinterpret_cast<const uint2*>(xr), xv[u]);
      } else {
        const uint32_t raw = *reinterpret_cast<const uint32_t*>(xr);
        xv[u][0] = __uint_as_float(raw << 16); xv[u][1] = __uint_as_float(raw & 0xffff0000u);
      }
      if constexpr (E == 4) {
        unpack_bf16x4(*reinterpret_cast<const uint2*>(zr), zv[u]);
      } else {
        const uint32_t raw = *reinterpret_cast<const uint32_t*>(zr);
        zv[u][0] = __uint_as_float(raw << 16); zv[u][1] = __uint_as_float(raw & 0xffff0000u);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (!live[u]) continue;
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < E; ++i) {
        if (gate_first) xv[u][i] *= silu(zv[u][i]);
        ss += xv[u][i] * xv[u][i];
      }
      ss = warp_sum(ss);
      const float rinv = rsqrtf(ss * (1.0f / D) + eps);
      float out[E];
#pragma unroll
      for (int i = 0; i < E; ++i) {
        const float wv = w ? w[lane * E + i] : 1.0f;
        out[i] = xv[u][i] * rinv * wv * (gate_first ? 1.0f : silu(zv[u][i]));
      }
      if constexpr (E == 4) {
        const uint2 packed = make_uint2(pack_bf16x2(out[0], out[1]), pack_bf16x2(out[2], out[3]));
        if (n_peers > 0) {  // fused all-gather: the same row goes to every GPU's buffer (plain peer stores)
          for (int p = 0; p < n_peers; ++p)
            *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(peers[p])) + peer_off + yoff[u]) = packed;
        } else {
          *reinterpret_cast<uint2*>(y + yoff[u]) = packed;
        }
      } else {
        *reinterpret_cast<uint32_t*>(y + yoff[u]) = pack_bf16x2(out[0], out[1]);
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
  const int64_t blocks_needed = (rows + 7) / 8;  // 8 warps per block, one row per warp and pass
  const unsigned grid = (unsigned)(blocks_needed < 148 * 64 ? blocks_needed : 148 * 64);
  const int gate_first = (a.flags & AVE_GDN_FLAG_GATE_FIRST) ? 1 : 0;
  const __nv_bfloat16* z = reinterpret_cast<const __nv_bfloat16*>(a.z);
  __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(a.y);
  if (a.d == 128) {
    gated_rmsnorm_kernel<128, XT><<<grid, 256, 0, stream>>>(x, z, a.weight, y, rows, a.heads, a.x_stride_t, a.x_stride_h,
                                                            a.z_stride_t, a.z_stride_h, a.y_stride_t, a.y_stride_h, a.eps, gate_first, peers, n_peers, peer_off, nb);
  } else if (a.d == 64) {
    gated_rmsnorm_kernel<64, XT><<<grid, 256, 0, stream>>>(x, z, a.weight, y, rows, a.heads, a.x_stride_t, a.x_stride_h,
                                                           a.z_stride_t, a.z_stride_h, a.y_stride_t, a.y_stride_h, a.eps, gate_first, nullptr, 0, 0, nb);
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
