// Shared helpers for the GDN kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ave_gdn.h"

namespace ave {

extern thread_local int g_last_cuda_error;

inline int cuda_fail(cudaError_t e) {
  g_last_cuda_error = (int)e;
  return AVE_GDN_CUDA_ERROR;
}

#define AVE_CUDA_TRY(expr)                                   \
  do {                                                       \
    cudaError_t e__ = (expr);                                \
    if (e__ != cudaSuccess) return ::ave::cuda_fail(e__);    \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

__device__ __forceinline__ float bf2f(__nv_bfloat16 x) { return __bfloat162float(x); }

__device__ __forceinline__ void unpack_bf16x4(uint2 raw, float (&f)[4]) {
  // bf16 -> fp32 is a 16-bit shift
  f[0] = __uint_as_float(raw.x << 16);
  f[1] = __uint_as_float(raw.x & 0xffff0000u);
  f[2] = __uint_as_float(raw.y << 16);
  f[3] = __uint_as_float(raw.y & 0xffff0000u);
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&t);
}

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

// Butterfly reduction of 32 per-lane values over the 32 lanes: on return lane l holds the sum over all lanes of v[l].
__device__ __forceinline__ float reduce32(float (&v)[32], int lane) {
#pragma unroll
  for (int s = 16, n = 32; s >= 1; s >>= 1, n >>= 1) {
    const bool upper = (lane & s) != 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      if (i < n / 2) {
        const float send = upper ? v[i] : v[i + n / 2];
        const float keep = upper ? v[i + n / 2] : v[i];
        v[i] = keep + __shfl_xor_sync(0xffffffffu, send, s);
      }
    }
  }
  return v[0];
}

__device__ __forceinline__ float silu(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

// silu of two values with the multiplies and the add as packed fp32 pairs (one instruction per pair); the exponential
// and the reciprocal stay scalar special-function operations
__device__ __forceinline__ float2 silu2(float2 x) {
  const float2 t = __fmul2_rn(x, make_float2(-1.4426950408889634f, -1.4426950408889634f));
  float2 e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.x) : "f"(t.x));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.y) : "f"(t.y));
  const float2 d = __ffma2_rn(e, make_float2(1.f, 1.f), make_float2(1.f, 1.f));
  float2 r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r.x) : "f"(d.x));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r.y) : "f"(d.y));
  return __fmul2_rn(x, r);
}
// two bf16 values packed in 32 bits -> fp32 pair (a 16-bit shift and a mask)
__device__ __forceinline__ float2 bf16x2_to_float2(uint32_t raw) {
  return make_float2(__uint_as_float(raw << 16), __uint_as_float(raw & 0xffff0000u));
}

// Sequence n of a dense [B,T] batch or of a packed varlen batch: batch row, first token, length.
struct SeqSpan {
  int b;
  int t0;
  int len;
  bool ok;
};

__device__ __forceinline__ SeqSpan seq_span(const int32_t* cu_seqlens, int n, int T, uint32_t* status) {
  SeqSpan s;
  if (cu_seqlens == nullptr) {
    s.b = n; s.t0 = 0; s.len = T; s.ok = true;
    return s;
  }
  const int a = cu_seqlens[n], e = cu_seqlens[n + 1];
  s.b = 0; s.t0 = a; s.len = e - a;
  s.ok = (a >= 0) && (e >= a) && (e <= T);
  if (!s.ok) {
    if (status != nullptr && threadIdx.x == 0) atomicOr(status, AVE_GDN_DEV_BAD_SEQLEN);
    s.len = 0;
  }
  return s;
}

}  // namespace ave
