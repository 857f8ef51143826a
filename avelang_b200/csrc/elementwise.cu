// Bandwidth-bound helpers around the recurrence: depthwise causal conv1d + SiLU, and the gate/beta math.
#include "common.cuh"

namespace ave {

// One thread owns 8 adjacent channels (one 16-byte load per token) and walks a run of tokens with the
// last width-1 inputs held in registers, so each input element is read from HBM once per run (+ halo).
// The kernel is bound by instruction issue, not by HBM (about 6 bytes cross the memory system per warp instruction
// the SMs can issue), so the arithmetic runs on packed fp32 pairs: one FFMA2 per tap and channel pair.
template <int WIDTH>
__global__ void __launch_bounds__(128) conv1d_silu_kernel(const AveConvArgs a, int tokens_per_cta) {
  const int cg = blockIdx.x * blockDim.x + threadIdx.x;  // channel group
  if (cg * 8 >= a.C) return;
  const int b = blockIdx.z;
  const int t_begin = blockIdx.y * tokens_per_cta;
  const int t_end = min(a.T, t_begin + tokens_per_cta);
  if (t_begin >= t_end) return;
  const __nv_bfloat16* xg = reinterpret_cast<const __nv_bfloat16*>(a.x) + b * a.x_stride_b + cg * 8;
  __nv_bfloat16* yg = reinterpret_cast<__nv_bfloat16*>(a.y) + b * a.y_stride_b + cg * 8;

  float2 w[4][WIDTH], bias[4];  // channel pairs
  {
    const __nv_bfloat16* wg = reinterpret_cast<const __nv_bfloat16*>(a.w) + (int64_t)cg * 8 * WIDTH;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
#pragma unroll
      for (int j = 0; j < WIDTH; ++j) w[c][j] = make_float2(bf2f(wg[(2 * c) * WIDTH + j]), bf2f(wg[(2 * c + 1) * WIDTH + j]));
      bias[c] = a.bias ? make_float2(bf2f(reinterpret_cast<const __nv_bfloat16*>(a.bias)[cg * 8 + 2 * c]),
                                     bf2f(reinterpret_cast<const __nv_bfloat16*>(a.bias)[cg * 8 + 2 * c + 1]))
                       : make_float2(0.f, 0.f);
    }
  }
  // sequence containing t_begin
  int seq = 0, seq_start = 0, seq_end = a.T;
  if (a.cu_seqlens != nullptr) {
    int lo = 0, hi = a.n_seqs;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (a.cu_seqlens[mid] <= t_begin) lo = mid; else hi = mid;
    }
    seq = lo; seq_start = a.cu_seqlens[seq]; seq_end = a.cu_seqlens[seq + 1];
  }
  auto unpack = [](uint4 raw, float2 (&f)[4]) {
    f[0] = bf16x2_to_float2(raw.x); f[1] = bf16x2_to_float2(raw.y);
    f[2] = bf16x2_to_float2(raw.z); f[3] = bf16x2_to_float2(raw.w);
  };
  float2 hist[WIDTH][4];  // hist[WIDTH-1] is the current token
#pragma unroll
  for (int j = 0; j < WIDTH - 1; ++j) {
    const int t = t_begin - (WIDTH - 1) + j;
    if (t >= seq_start && t >= 0) {
      unpack(*reinterpret_cast<const uint4*>(xg + (int64_t)t * a.x_stride_t), hist[j]);
    } else {
#pragma unroll
      for (int c = 0; c < 4; ++c) hist[j][c] = make_float2(0.f, 0.f);
    }
  }
  const __nv_bfloat16* xp = xg + (int64_t)t_begin * a.x_stride_t;
  __nv_bfloat16* yp = yg + (int64_t)t_begin * a.y_stride_t;
  // tokens are fetched eight at a time so that eight 16-byte loads are in flight per thread
  for (int tb = t_begin; tb < t_end; tb += 8) {
    uint4 raw[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      raw[j] = (tb + j < t_end) ? *reinterpret_cast<const uint4*>(xp + (int64_t)j * a.x_stride_t) : make_uint4(0u, 0u, 0u, 0u);
    xp += 8 * a.x_stride_t;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int t = tb + j;
      if (t >= t_end) break;
      if (a.cu_seqlens != nullptr && t >= seq_end) {  // crossed into the next sequence: forget history
        while (t >= seq_end && seq + 1 < a.n_seqs) { ++seq; seq_start = seq_end; seq_end = a.cu_seqlens[seq + 1]; }
#pragma unroll
        for (int jj = 0; jj < WIDTH - 1; ++jj)
#pragma unroll
          for (int c = 0; c < 4; ++c) hist[jj][c] = make_float2(0.f, 0.f);
      }
      unpack(raw[j], hist[WIDTH - 1]);
      uint32_t packed[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float2 acc = bias[c];
#pragma unroll
        for (int jj = 0; jj < WIDTH; ++jj) acc = __ffma2_rn(w[c][jj], hist[jj][c], acc);
        const float2 o = silu2(acc);
        packed[c] = pack_bf16x2(o.x, o.y);
      }
      *reinterpret_cast<uint4*>(yp) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      yp += a.y_stride_t;
#pragma unroll
      for (int jj = 0; jj < WIDTH - 1; ++jj)
#pragma unroll
        for (int c = 0; c < 4; ++c) hist[jj][c] = hist[jj + 1][c];
    }
  }
}

int launch_conv1d_silu(const AveConvArgs& a, cudaStream_t stream) {
  if (a.B == 0 || a.T == 0 || a.C == 0) return AVE_GDN_OK;
  const int groups = a.C / 8;
  const int threads = 128;
  const int tokens_per_cta = 64;
  dim3 grid((groups + threads - 1) / threads, (a.T + tokens_per_cta - 1) / tokens_per_cta, a.B);
  switch (a.width) {
    case 2: conv1d_silu_kernel<2><<<grid, threads, 0, stream>>>(a, tokens_per_cta); break;
    case 3: conv1d_silu_kernel<3><<<grid, threads, 0, stream>>>(a, tokens_per_cta); break;
    case 4: conv1d_silu_kernel<4><<<grid, threads, 0, stream>>>(a, tokens_per_cta); break;
    default: return AVE_GDN_UNSUPPORTED;
  }
  AVE_CUDA_TRY(cudaGetLastError());
  return AVE_GDN_OK;
}

// Decode-time convolution: one thread per (sequence, 8 channels); history rows are channel-contiguous, so every access
// is a coalesced 16-byte piece.
template <int WIDTH>
__global__ void __launch_bounds__(128) conv1d_update_kernel(const AveConvUpdateArgs a) {
  const int cg = blockIdx.x * blockDim.x + threadIdx.x;
  const int n = blockIdx.y;
  if (cg * 8 >= a.C) return;
  int slot = a.state_indices ? a.state_indices[n] : n;
  if (slot >= a.num_slots) {
    if (a.status != nullptr && threadIdx.x == 0 && blockIdx.x == 0) atomicOr(a.status, AVE_GDN_DEV_BAD_SLOT);
    return;
  }
  if (slot < 0) return;
  __nv_bfloat16* st = reinterpret_cast<__nv_bfloat16*>(a.conv_state) + (int64_t)slot * (WIDTH - 1) * a.C + cg * 8;
  auto unpack8 = [](uint4 raw, float (&f)[8]) {
    f[0] = __uint_as_float(raw.x << 16); f[1] = __uint_as_float(raw.x & 0xffff0000u);
    f[2] = __uint_as_float(raw.y << 16); f[3] = __uint_as_float(raw.y & 0xffff0000u);
    f[4] = __uint_as_float(raw.z << 16); f[5] = __uint_as_float(raw.z & 0xffff0000u);
    f[6] = __uint_as_float(raw.w << 16); f[7] = __uint_as_float(raw.w & 0xffff0000u);
  };
  uint4 raw[WIDTH];
#pragma unroll
  for (int j = 0; j < WIDTH - 1; ++j) raw[j] = *reinterpret_cast<const uint4*>(st + (int64_t)j * a.C);
  raw[WIDTH - 1] = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(a.x) + n * a.x_stride + cg * 8);
  float acc[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) acc[c] = a.bias ? bf2f(reinterpret_cast<const __nv_bfloat16*>(a.bias)[cg * 8 + c]) : 0.f;
  const __nv_bfloat16* wg = reinterpret_cast<const __nv_bfloat16*>(a.w) + (int64_t)cg * 8 * WIDTH;
#pragma unroll
  for (int j = 0; j < WIDTH; ++j) {
    float xv[8];
    unpack8(raw[j], xv);
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[c] = fmaf(bf2f(wg[c * WIDTH + j]), xv[c], acc[c]);
  }
  uint4 packed = make_uint4(pack_bf16x2(silu(acc[0]), silu(acc[1])), pack_bf16x2(silu(acc[2]), silu(acc[3])),
                            pack_bf16x2(silu(acc[4]), silu(acc[5])), pack_bf16x2(silu(acc[6]), silu(acc[7])));
  *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.y) + n * a.y_stride + cg * 8) = packed;
#pragma unroll
  for (int j = 0; j < WIDTH - 1; ++j) *reinterpret_cast<uint4*>(st + (int64_t)j * a.C) = raw[j + 1];  // shift in the new token
}

int launch_conv1d_update(const AveConvUpdateArgs& a, cudaStream_t stream) {
  if (a.n_seqs == 0 || a.C == 0) return AVE_GDN_OK;
  dim3 grid((a.C / 8 + 127) / 128, a.n_seqs);
  switch (a.width) {
    case 2: conv1d_update_kernel<2><<<grid, 128, 0, stream>>>(a); break;
    case 3: conv1d_update_kernel<3><<<grid, 128, 0, stream>>>(a); break;
    case 4: conv1d_update_kernel<4><<<grid, 128, 0, stream>>>(a); break;
    default: return AVE_GDN_UNSUPPORTED;
  }
  AVE_CUDA_TRY(cudaGetLastError());
  return AVE_GDN_OK;
}

__global__ void __launch_bounds__(256) gate_beta_kernel(const AveGateArgs a) {
  const int64_t total = a.rows * a.Hv;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = e / a.Hv;
    const int h = (int)(e - r * a.Hv);
    const float av = bf2f(reinterpret_cast<const __nv_bfloat16*>(a.a)[r * a.a_stride_row + h]) + a.dt_bias[h];
    const float bv = bf2f(reinterpret_cast<const __nv_bfloat16*>(a.b)[r * a.b_stride_row + h]);
    const float sp = av > 20.f ? av : log1pf(expf(av));  // softplus
    a.g[e] = -expf(a.A_log[h]) * sp;
    a.beta[e] = 1.0f / (1.0f + expf(-bv));
  }
}

int launch_gate_beta(const AveGateArgs& a, cudaStream_t stream) {
  const int64_t total = a.rows * a.Hv;
  if (total == 0) return AVE_GDN_OK;
  const int64_t blocks = (total + 255) / 256;
  gate_beta_kernel<<<(unsigned)(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0, stream>>>(a);
  AVE_CUDA_TRY(cudaGetLastError());
  return AVE_GDN_OK;
}

}  // namespace ave
