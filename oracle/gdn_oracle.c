/* CPU checker for the gated-delta-net recurrence, in C.  TEST INFRASTRUCTURE ONLY:
 * it is never linked into, loaded by or called from the shipped library; the test-suite,
 * the smoke check and the benchmark's CPU-baseline leg use it as the checker / baseline.
 *
 * PARITY UNPINNED BY THE REFERENCE: the reference tree has no GDN code or vectors
 * (python/avelang_kernels/ holds only amdgpu_gemm.py).  This restates, token by token,
 *     M <- exp(g_t) M;  r = M^T k_t;  u = beta_t (v_t - r);  M <- M + k_t u^T;  o_t = scale M^T q_t
 * with M key-major [dk][dv], the transpose of the recurrence in the task's configuration text
 *     S_t = exp(g_t) S_{t-1} (I - beta_t k_t k_t^T) + beta_t v_t k_t^T,  o_t = scale S_t q_t.
 * It is validated against the Python derivations in gdn_oracle.py by the CPU test-suite.
 *
 * Layout: packed tokens [Ttot][H][d] (row stride given in elements), sequences by cu_seqlens[N+1],
 * states [N][Hv][dk][dv].  Inputs are fp32 arrays (bf16 values already widened by the caller).
 * Built twice: REAL=double (parity checker) and REAL=float (CPU baseline).  OpenMP over (seq, head). */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifndef REAL
#define REAL double
#endif
#define CAT_(a, b) a##b
#define CAT(a, b) CAT_(a, b)
#define FN(name) CAT(name, SUFFIX)

int FN(gdn_oracle_recurrent_)(const float* q, const float* k, const float* v, const float* g,
                              const float* beta, const float* s0, float* o, float* sT,
                              const int32_t* cu_seqlens, int32_t n_seqs, int32_t Hk, int32_t Hv,
                              int32_t dk, int32_t dv, int64_t q_row, int64_t k_row, int64_t v_row,
                              int64_t o_row, int64_t g_row, float scale, int32_t l2norm_qk) {
  const int rep = Hv / Hk;
  int rc = 0;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
  for (int n = 0; n < n_seqs; ++n) {
    for (int h = 0; h < Hv; ++h) {
      REAL* M = (REAL*)malloc(sizeof(REAL) * dk * dv);
      REAL* u = (REAL*)malloc(sizeof(REAL) * dv);
      REAL* kk = (REAL*)malloc(sizeof(REAL) * dk);
      REAL* qq = (REAL*)malloc(sizeof(REAL) * dk);
      REAL* acc = (REAL*)malloc(sizeof(REAL) * dv);
      if (!M || !u || !kk || !qq || !acc) { rc = 1; free(M); free(u); free(kk); free(qq); free(acc); continue; }
      const int hk = h / rep;
      for (int i = 0; i < dk * dv; ++i)
        M[i] = s0 ? (REAL)s0[((int64_t)n * Hv + h) * dk * dv + i] : (REAL)0;
      for (int64_t t = cu_seqlens[n]; t < cu_seqlens[n + 1]; ++t) {
        const float* kt = k + t * k_row + (int64_t)hk * dk;
        const float* qt = q + t * q_row + (int64_t)hk * dk;
        const float* vt = v + t * v_row + (int64_t)h * dv;
        float* ot = o + t * o_row + (int64_t)h * dv;
        REAL kn = 1, qn = 1;
        if (l2norm_qk) {
          REAL sk = 0, sq = 0;
          for (int i = 0; i < dk; ++i) { sk += (REAL)kt[i] * kt[i]; sq += (REAL)qt[i] * qt[i]; }
          kn = 1 / sqrt(sk + (REAL)1e-6); qn = 1 / sqrt(sq + (REAL)1e-6);
        }
        for (int i = 0; i < dk; ++i) { kk[i] = (REAL)kt[i] * kn; qq[i] = (REAL)qt[i] * qn; }
        const REAL a = exp((REAL)g[t * g_row + h]);
        const REAL b = (REAL)beta[t * g_row + h];
        for (int j = 0; j < dv; ++j) u[j] = 0;
        for (int i = 0; i < dk; ++i) {           /* decay, and r = M^T k on the decayed state */
          REAL* Mi = M + (int64_t)i * dv;
          const REAL ki = kk[i];
          for (int j = 0; j < dv; ++j) { Mi[j] *= a; u[j] += Mi[j] * ki; }
        }
        for (int j = 0; j < dv; ++j) u[j] = b * ((REAL)vt[j] - u[j]);
        for (int j = 0; j < dv; ++j) acc[j] = 0;
        for (int i = 0; i < dk; ++i) {           /* rank-1 update, and o = M^T q on the new state */
          REAL* Mi = M + (int64_t)i * dv;
          const REAL ki = kk[i], qi = qq[i];
          for (int j = 0; j < dv; ++j) { Mi[j] += ki * u[j]; acc[j] += Mi[j] * qi; }
        }
        for (int j = 0; j < dv; ++j) ot[j] = (float)((REAL)scale * acc[j]);
      }
      if (sT)
        for (int i = 0; i < dk * dv; ++i) sT[((int64_t)n * Hv + h) * dk * dv + i] = (float)M[i];
      free(M); free(u); free(kk); free(qq); free(acc);
    }
  }
  return rc;
}
