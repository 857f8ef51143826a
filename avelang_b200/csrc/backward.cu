// Backward pass of the gated delta rule (d_k = d_v = 128), token by token in reverse, fp32 on the CUDA cores.
//
// Forward, per token (M is the key-major state [dk][dv], a = exp(g)):
//     Mb = a M;   r = Mb^T k;   u = beta (v - r);   M' = Mb + k u^T;   o = scale M'^T q
// Backward, given do and the gradient dM' that flows in from the future:
//     dM' += scale q do^T;          dq = scale M' do
//     du = dM'^T k;                 dk = dM' u + Mb dr        (dr = -beta du)
//     dbeta = du . (v - r);         dv = beta du
//     dMb = dM' + k dr^T;           dg = <dMb, Mb>;           dM = a dMb
// so the reverse sweep needs Mb of every token.  One CTA walks one (sequence, value head): a forward sweep leaves the
// state at every 64-token boundary in the checkpoint area; then, chunk by chunk from the end, the chunk's 64 Mb tiles
// are recomputed from its checkpoint into a per-CTA scratch ring and consumed in reverse.  The state tile and its
// gradient stay in registers (a warp owns 16 rows, a lane 4 columns); column reductions (r, du) cross warps through
// shared memory, row reductions (dq, dk) are one 32-value butterfly per warp and token.
// This is the correct-first form of the pass: every token costs a 64 KiB tile written and read back, and a handful of
// CTA barriers; a chunked (WY) backward on the tensor cores is the faster successor.
#include "common.cuh"

namespace ave {
namespace {

constexpr int BD = 128, BW = 8, BROWS = BD / BW, BCH = 64;  // head dim, warps, rows per warp, tokens per checkpoint

struct Tok {
  float alpha, beta;
  float v4[4], do4[4];
};

__global__ void __launch_bounds__(256, 1) gdn_backward_kernel(const AveGdnBwdArgs a, int n_units) {
  __shared__ __align__(16) float k_s[BD];
  __shared__ __align__(16) float q_s[BD];
  __shared__ __align__(16) float red[2][BW][BD];
  __shared__ float red_g[BW];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int col = lane * 4, row0 = warp * BROWS;
  const int r_heads = a.Hv / a.Hk;
  float* ckpt = reinterpret_cast<float*>(a.workspace);
  const int64_t ckpt_tiles = ((int64_t)a.B * a.T / BCH + a.n_seqs + 1) * a.Hv;
  float* ring = ckpt + ckpt_tiles * (int64_t)(BD * BD) + (int64_t)blockIdx.x * BCH * (int64_t)(BD * BD);  // this CTA's 64 tiles

  for (int unit = blockIdx.x; unit < n_units; unit += gridDim.x) {
    const int n = unit / a.Hv, h = unit % a.Hv, hk = h / r_heads;
    const SeqSpan sp = seq_span(a.cu_seqlens, n, a.T, a.status);
    if (!sp.ok || sp.len == 0) {
      if (sp.ok && a.d_initial_state != nullptr) {  // empty sequence: the state gradient passes through
        const int64_t tile = ((int64_t)n * a.Hv + h) * (int64_t)(BD * BD);
        for (int e = tid; e < BD * BD; e += 256) a.d_initial_state[tile + e] = a.d_final_state ? a.d_final_state[tile + e] : 0.f;
      }
      continue;
    }
    const int64_t tile = ((int64_t)n * a.Hv + h) * (int64_t)(BD * BD);
    const __nv_bfloat16* q_base = reinterpret_cast<const __nv_bfloat16*>(a.q) + sp.b * a.q_stride_b + (int64_t)hk * a.q_stride_h;
    const __nv_bfloat16* k_base = reinterpret_cast<const __nv_bfloat16*>(a.k) + sp.b * a.k_stride_b + (int64_t)hk * a.k_stride_h;
    const __nv_bfloat16* v_base = reinterpret_cast<const __nv_bfloat16*>(a.v) + sp.b * a.v_stride_b + (int64_t)h * a.v_stride_h;
    const __nv_bfloat16* do_base = reinterpret_cast<const __nv_bfloat16*>(a.d_o) + sp.b * a.do_stride_b + (int64_t)h * a.do_stride_h;
    const float* g_base = a.g + sp.b * a.g_stride_b + h;
    const float* beta_base = a.beta + sp.b * a.g_stride_b + h;
    const int n_chunks = (sp.len + BCH - 1) / BCH;
    auto ckpt_of = [&](int j) {  // unique per (sequence, chunk): chunks of later sequences get later indices
      return ckpt + ((((int64_t)sp.b * a.T + sp.t0 + j * BCH) / BCH + n) * a.Hv + h) * (int64_t)(BD * BD);
    };
    // vectors of token `tok` into shared memory / registers; the caller synchronises
    auto load_token = [&](int64_t tok, Tok& tk, bool need_q) {
      if (tid < BD) k_s[tid] = bf2f(k_base[tok * a.k_stride_t + tid]);
      else if (need_q) q_s[tid - BD] = bf2f(q_base[tok * a.q_stride_t + tid - BD]);
      unpack_bf16x4(*reinterpret_cast<const uint2*>(v_base + tok * a.v_stride_t + col), tk.v4);
      if (need_q) unpack_bf16x4(*reinterpret_cast<const uint2*>(do_base + tok * a.do_stride_t + col), tk.do4);
      tk.alpha = __expf(g_base[tok * a.g_stride_t]);
      tk.beta = beta_base[tok * a.g_stride_t];
    };
    // column reduction over the 128 rows of per-thread partials p (this thread's 16 rows): total per column, in all threads
    auto col_reduce = [&](int which, const float (&p)[4], float (&out)[4]) {
      *reinterpret_cast<float4*>(&red[which][warp][col]) = make_float4(p[0], p[1], p[2], p[3]);
      __syncthreads();
      float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int w = 0; w < BW; ++w) {
        const float4 x = *reinterpret_cast<const float4*>(&red[which][w][col]);
        s.x += x.x; s.y += x.y; s.z += x.z; s.w += x.w;
      }
      out[0] = s.x; out[1] = s.y; out[2] = s.z; out[3] = s.w;
    };
    // one forward token on the state in registers: S <- Mb = a S (optionally stored), then S <- Mb + k u^T
    float4 S[BROWS];
    auto forward_token = [&](int64_t tok, float* store_mb) {
      Tok tk;
      __syncthreads();  // the shared vectors of the previous token are no longer read
      load_token(tok, tk, false);
      __syncthreads();
      float p[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < BROWS; ++i) {
        S[i].x *= tk.alpha; S[i].y *= tk.alpha; S[i].z *= tk.alpha; S[i].w *= tk.alpha;
        if (store_mb != nullptr) *reinterpret_cast<float4*>(store_mb + (row0 + i) * BD + col) = S[i];
        const float kr = k_s[row0 + i];
        p[0] += S[i].x * kr; p[1] += S[i].y * kr; p[2] += S[i].z * kr; p[3] += S[i].w * kr;
      }
      float r[4];
      col_reduce(0, p, r);
      float u[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) u[c] = tk.beta * (tk.v4[c] - r[c]);
#pragma unroll
      for (int i = 0; i < BROWS; ++i) {
        const float kr = k_s[row0 + i];
        S[i].x += kr * u[0]; S[i].y += kr * u[1]; S[i].z += kr * u[2]; S[i].w += kr * u[3];
      }
    };

    // ---- forward sweep: checkpoints at every chunk boundary
    {
      const float* s0 = a.initial_state ? a.initial_state + tile : nullptr;
#pragma unroll
      for (int i = 0; i < BROWS; ++i)
        S[i] = s0 ? *reinterpret_cast<const float4*>(s0 + (row0 + i) * BD + col) : make_float4(0.f, 0.f, 0.f, 0.f);
      for (int j = 0; j < n_chunks; ++j) {
        float* dst = ckpt_of(j);
#pragma unroll
        for (int i = 0; i < BROWS; ++i) *reinterpret_cast<float4*>(dst + (row0 + i) * BD + col) = S[i];
        if (j == n_chunks - 1) break;  // the last chunk is recomputed below anyway
        for (int t = 0; t < BCH; ++t) forward_token(sp.t0 + j * BCH + t, nullptr);
      }
    }

    // ---- reverse sweep
    float4 dM[BROWS];
    {
      const float* ds = a.d_final_state ? a.d_final_state + tile : nullptr;
#pragma unroll
      for (int i = 0; i < BROWS; ++i)
        dM[i] = ds ? *reinterpret_cast<const float4*>(ds + (row0 + i) * BD + col) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int j = n_chunks - 1; j >= 0; --j) {
      const int len = min(BCH, sp.len - j * BCH);
      const float* src = ckpt_of(j);
#pragma unroll
      for (int i = 0; i < BROWS; ++i) S[i] = *reinterpret_cast<const float4*>(src + (row0 + i) * BD + col);
      for (int t = 0; t < len; ++t) forward_token(sp.t0 + j * BCH + t, ring + (int64_t)t * (BD * BD));
      // every thread re-reads only the tile elements it wrote itself, so no fence is needed around the ring
      for (int t = len - 1; t >= 0; --t) {
        const int64_t tok = sp.t0 + j * BCH + t;
        const float* mb = ring + (int64_t)t * (BD * BD);
        Tok tk;
        __syncthreads();
        load_token(tok, tk, true);
#pragma unroll
        for (int i = 0; i < BROWS; ++i) S[i] = *reinterpret_cast<const float4*>(mb + (row0 + i) * BD + col);  // Mb of this token
        __syncthreads();
        // r = Mb^T k, u = beta (v - r)
        float p[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < BROWS; ++i) {
          const float kr = k_s[row0 + i];
          p[0] += S[i].x * kr; p[1] += S[i].y * kr; p[2] += S[i].z * kr; p[3] += S[i].w * kr;
        }
        float r[4], u[4], vr[4];
        col_reduce(0, p, r);
#pragma unroll
        for (int c = 0; c < 4; ++c) { vr[c] = tk.v4[c] - r[c]; u[c] = tk.beta * vr[c]; }
        // dM' += scale q do^T;  rows of dq = scale M' do and the first half of dk = dM' u;  du = dM'^T k
        float rowv[32];
        float pu[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < BROWS; ++i) {
          const float kr = k_s[row0 + i], qs = a.scale * q_s[row0 + i];
          dM[i].x += qs * tk.do4[0]; dM[i].y += qs * tk.do4[1]; dM[i].z += qs * tk.do4[2]; dM[i].w += qs * tk.do4[3];
          const float m0 = S[i].x + kr * u[0], m1 = S[i].y + kr * u[1], m2 = S[i].z + kr * u[2], m3 = S[i].w + kr * u[3];
          rowv[i] = a.scale * (m0 * tk.do4[0] + m1 * tk.do4[1] + m2 * tk.do4[2] + m3 * tk.do4[3]);
          rowv[16 + i] = dM[i].x * u[0] + dM[i].y * u[1] + dM[i].z * u[2] + dM[i].w * u[3];
          pu[0] += dM[i].x * kr; pu[1] += dM[i].y * kr; pu[2] += dM[i].z * kr; pu[3] += dM[i].w * kr;
        }
        float du[4], dr[4];
        col_reduce(1, pu, du);
#pragma unroll
        for (int c = 0; c < 4; ++c) dr[c] = -tk.beta * du[c];
        // dMb = dM' + k dr^T;  second half of dk = Mb dr;  dg = <dMb, Mb>;  dM = a dMb
        float gpart = 0.f;
#pragma unroll
        for (int i = 0; i < BROWS; ++i) {
          const float kr = k_s[row0 + i];
          rowv[16 + i] += S[i].x * dr[0] + S[i].y * dr[1] + S[i].z * dr[2] + S[i].w * dr[3];
          dM[i].x += kr * dr[0]; dM[i].y += kr * dr[1]; dM[i].z += kr * dr[2]; dM[i].w += kr * dr[3];
          gpart += dM[i].x * S[i].x + dM[i].y * S[i].y + dM[i].z * S[i].z + dM[i].w * S[i].w;
          dM[i].x *= tk.alpha; dM[i].y *= tk.alpha; dM[i].z *= tk.alpha; dM[i].w *= tk.alpha;
        }
        const float rowsum = reduce32(rowv, lane);  // lanes 0..15: dq of rows row0 + lane; lanes 16..31: dk of rows row0 + lane - 16
        const int64_t kq_off = (((int64_t)sp.b * a.T + tok) * a.Hv + h) * BD + row0 + (lane & 15);
        if (lane < 16) a.d_q[kq_off] = rowsum; else a.d_k[kq_off] = rowsum;
        gpart = warp_sum(gpart);
        if (lane == 0) red_g[warp] = gpart;
        if (warp == 0) {  // every warp holds every column once; warp 0 writes the per-column and per-token results
          float db = du[0] * vr[0] + du[1] * vr[1] + du[2] * vr[2] + du[3] * vr[3];
          db = warp_sum(db);
          const int64_t v_off = (((int64_t)sp.b * a.T + tok) * a.Hv + h) * BD + col;
          *reinterpret_cast<float4*>(a.d_v + v_off) = make_float4(tk.beta * du[0], tk.beta * du[1], tk.beta * du[2], tk.beta * du[3]);
          if (lane == 0) a.d_beta[((int64_t)sp.b * a.T + tok) * a.Hv + h] = db;
        }
        __syncthreads();
        if (tid == 0) {
          float gs = 0.f;
#pragma unroll
          for (int w = 0; w < BW; ++w) gs += red_g[w];
          a.d_g[((int64_t)sp.b * a.T + tok) * a.Hv + h] = gs;
        }
      }
    }
    if (a.d_initial_state != nullptr) {
      float* dst = a.d_initial_state + tile;
#pragma unroll
      for (int i = 0; i < BROWS; ++i) *reinterpret_cast<float4*>(dst + (row0 + i) * BD + col) = dM[i];
    }
  }
}

int backward_grid(const AveGdnBwdArgs& a) {
  const int64_t units = (int64_t)a.n_seqs * a.Hv;
  return (int)(units < 148 ? units : 148);
}

}  // namespace

size_t backward_workspace_bytes(const AveGdnBwdArgs& a) {
  const size_t tile = (size_t)BD * BD * 4;
  const size_t ckpt = ((size_t)a.B * a.T / BCH + (size_t)a.n_seqs + 1) * (size_t)a.Hv * tile;
  return ckpt + (size_t)backward_grid(a) * BCH * tile;
}

int launch_backward(const AveGdnBwdArgs& a, cudaStream_t stream) {
  const int units = a.n_seqs * a.Hv;
  if (units == 0 || a.T == 0) return AVE_GDN_OK;
  gdn_backward_kernel<<<backward_grid(a), 256, 0, stream>>>(a, units);
  AVE_CUDA_TRY(cudaGetLastError());
  return AVE_GDN_OK;
}

}  // namespace ave
