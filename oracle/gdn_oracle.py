"""CPU checker for the gated-delta-net (GDN) path.  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package may import this file: only the test-suite, the
smoke check and the CPU-baseline leg of the benchmark use it, and only as the
checker, never as the thing measured as the product.

PARITY UNPINNED BY THE REFERENCE.  The reference project's mounted tree has no
GDN code (python/avelang_kernels/ holds only amdgpu_gemm.py), hence no golden
vectors, known-answer tests or fixtures for this path.  This file restates the
recurrence published in the task's configuration text:

    S_t = exp(g_t) * S_{t-1} (I - beta_t k_t k_t^T) + beta_t v_t k_t^T
    o_t = scale * S_t^T-applied-to q_t

stored key-major (M = S^T, shape [dk, dv]):

    M <- exp(g_t) M;  r = M^T k_t;  u = beta_t (v_t - r);  M <- M + k_t u^T;
    o_t = scale * M^T q_t

What pins it instead: (1) three independent derivations in this file (token
recurrence, chunked WY/UT form, affine chunk-summary form) that must agree to
1e-12 in fp64; (2) the C restatement in gdn_oracle.c; (3) an optional
import-only cross-check against a third-party package when it is installed.
The style (seeded randn inputs, a PyTorch expression as the checker) follows
the reference's own tests, test/examples/gemm/amdgpu/test_amdgpu_gemm.py:15-31.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def _expand_heads(x: torch.Tensor, Hv: int) -> torch.Tensor:
    """[.., Hk, d] -> [.., Hv, d]; value head h reads key head h // (Hv/Hk)."""
    Hk = x.shape[-2]
    if Hk == Hv:
        return x
    return x.repeat_interleave(Hv // Hk, dim=-2)


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """x / sqrt(sum(x^2) + eps) over the last dim, in the dtype of x."""
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + eps)


def _seq_bounds(B, T, cu_seqlens):
    if cu_seqlens is None:
        return [(b, 0, T) for b in range(B)]
    cu = [int(c) for c in cu_seqlens.tolist()]
    return [(0, cu[i], cu[i + 1]) for i in range(len(cu) - 1)]


def naive_recurrent_gated_delta_rule(q, k, v, g, beta, scale=None, initial_state=None,
                                     cu_seqlens=None, dtype=torch.float64,
                                     use_qk_l2norm_in_kernel=False):
    """Token-by-token recurrence; accumulates in ``dtype`` (fp32 = CPU baseline,
    fp64 = parity checker).  Returns (o [B,T,Hv,dv], final_state [N,Hv,dk,dv]) in ``dtype``."""
    B, T, Hk, dk = q.shape
    Hv, dv = v.shape[-2], v.shape[-1]
    scale = dk ** -0.5 if scale is None else scale
    q, k, v, g, beta = (x.to(dtype) for x in (q, k, v, g, beta))
    if use_qk_l2norm_in_kernel:
        q, k = l2norm(q), l2norm(k)
    q, k = _expand_heads(q, Hv), _expand_heads(k, Hv)
    seqs = _seq_bounds(B, T, cu_seqlens)
    o = torch.zeros(B, T, Hv, dv, dtype=dtype)
    final = torch.zeros(len(seqs), Hv, dk, dv, dtype=dtype)
    for n, (b, t0, t1) in enumerate(seqs):
        M = torch.zeros(Hv, dk, dv, dtype=dtype) if initial_state is None else initial_state[n].to(dtype).clone()
        for t in range(t0, t1):
            kt, qt, vt = k[b, t], q[b, t], v[b, t]
            M = M * torch.exp(g[b, t])[:, None, None]
            r = torch.einsum("hkv,hk->hv", M, kt)
            u = beta[b, t][:, None] * (vt - r)
            M = M + kt[:, :, None] * u[:, None, :]
            o[b, t] = scale * torch.einsum("hkv,hk->hv", M, qt)
        final[n] = M
    return o, final


def chunk_gated_delta_rule_ref(q, k, v, g, beta, scale=None, initial_state=None, cu_seqlens=None,
                               dtype=torch.float64, chunk=64):
    """Chunked WY/UT form, an independent derivation of the same function.

    Per chunk with incoming state M0 and in-chunk cumulative gate b:
      A = strict_lower(beta_i e^{b_i-b_j} k_i.k_j);  T = (I+A)^-1
      W = T diag(beta e^b) K;  U = T diag(beta) V;  Vn = U - W M0
      O = scale (diag(e^b) Q M0 + lower_incl(e^{b_i-b_j} q_i.k_j) Vn)
      M1 = e^{b_C} M0 + K^T diag(e^{b_C-b}) Vn
    Only non-positive exponents are exponentiated."""
    B, T, Hk, dk = q.shape
    Hv, dv = v.shape[-2], v.shape[-1]
    scale = dk ** -0.5 if scale is None else scale
    q, k, v, g, beta = (x.to(dtype) for x in (q, k, v, g, beta))
    q, k = _expand_heads(q, Hv), _expand_heads(k, Hv)
    seqs = _seq_bounds(B, T, cu_seqlens)
    o = torch.zeros(B, T, Hv, dv, dtype=dtype)
    final = torch.zeros(len(seqs), Hv, dk, dv, dtype=dtype)
    for n, (bi, t0, t1) in enumerate(seqs):
        M = torch.zeros(Hv, dk, dv, dtype=dtype) if initial_state is None else initial_state[n].to(dtype).clone()
        for c0 in range(t0, t1, chunk):
            c1 = min(c0 + chunk, t1)
            C = c1 - c0
            K = k[bi, c0:c1].transpose(0, 1)   # [Hv, C, dk]
            Q = q[bi, c0:c1].transpose(0, 1)
            V = v[bi, c0:c1].transpose(0, 1)
            bt = beta[bi, c0:c1].transpose(0, 1)  # [Hv, C]
            bcum = g[bi, c0:c1].transpose(0, 1).cumsum(-1)
            diff = bcum[:, :, None] - bcum[:, None, :]
            low_incl = torch.tril(torch.ones(C, C, dtype=torch.bool))
            D = torch.where(low_incl, torch.exp(torch.where(low_incl, diff, torch.zeros_like(diff))),
                            torch.zeros_like(diff))
            A = torch.tril(bt[:, :, None] * D * (K @ K.transpose(1, 2)), diagonal=-1)
            Tm = torch.linalg.solve_triangular(torch.eye(C, dtype=dtype) + A,
                                               torch.eye(C, dtype=dtype).expand(Hv, C, C), upper=False)
            W = Tm @ (K * (bt * torch.exp(bcum))[:, :, None])
            U = Tm @ (V * bt[:, :, None])
            Vn = U - W @ M
            P = D * (Q @ K.transpose(1, 2))
            O = scale * ((Q * torch.exp(bcum)[:, :, None]) @ M + P @ Vn)
            o[bi, c0:c1] = O.transpose(0, 1)
            bC = bcum[:, -1]
            M = torch.exp(bC)[:, None, None] * M + K.transpose(1, 2) @ (Vn * torch.exp(bC[:, None] - bcum)[:, :, None])
        final[n] = M
    return o, final


def affine_gated_delta_rule_ref(q, k, v, g, beta, scale=None, initial_state=None,
                                dtype=torch.float64, chunk=64):
    """Affine chunk-summary form (third derivation): every chunk is reduced to
    (Phi, Psi) with M1 = Phi M0 + Psi, O = scale (Qt M0 + P U).  Batch layout only."""
    B, T, Hk, dk = q.shape
    Hv, dv = v.shape[-2], v.shape[-1]
    scale = dk ** -0.5 if scale is None else scale
    q, k, v, g, beta = (x.to(dtype) for x in (q, k, v, g, beta))
    q, k = _expand_heads(q, Hv), _expand_heads(k, Hv)
    o = torch.zeros(B, T, Hv, dv, dtype=dtype)
    final = torch.zeros(B, Hv, dk, dv, dtype=dtype)
    for bi in range(B):
        M = torch.zeros(Hv, dk, dv, dtype=dtype) if initial_state is None else initial_state[bi].to(dtype).clone()
        for c0 in range(0, T, chunk):
            c1 = min(c0 + chunk, T)
            C = c1 - c0
            K = k[bi, c0:c1].transpose(0, 1)
            Q = q[bi, c0:c1].transpose(0, 1)
            V = v[bi, c0:c1].transpose(0, 1)
            bt = beta[bi, c0:c1].transpose(0, 1)
            bcum = g[bi, c0:c1].transpose(0, 1).cumsum(-1)
            low = torch.tril(torch.ones(C, C, dtype=torch.bool))
            diff = torch.where(low, bcum[:, :, None] - bcum[:, None, :], torch.zeros(Hv, C, C, dtype=dtype))
            D = torch.where(low, torch.exp(diff), torch.zeros_like(diff))
            A = torch.tril(bt[:, :, None] * D * (K @ K.transpose(1, 2)), diagonal=-1)
            Tm = torch.linalg.inv(torch.eye(C, dtype=dtype) + A)
            W = Tm @ (K * (bt * torch.exp(bcum))[:, :, None])
            U = Tm @ (V * bt[:, :, None])
            P = D * (Q @ K.transpose(1, 2))
            bC = bcum[:, -1]
            Kd = K * torch.exp(bC[:, None] - bcum)[:, :, None]
            Phi = torch.exp(bC)[:, None, None] * torch.eye(dk, dtype=dtype) - Kd.transpose(1, 2) @ W
            Psi = Kd.transpose(1, 2) @ U
            Qt = Q * torch.exp(bcum)[:, :, None] - P @ W
            o[bi, c0:c1] = (scale * (Qt @ M + P @ U)).transpose(0, 1)
            M = Phi @ M + Psi
        final[bi] = M
    return o, final


def gated_rmsnorm(x, z, weight=None, eps=1e-6, dtype=torch.float64):
    """y = w * x * rsqrt(mean(x^2) + eps) * silu(z) over the last dim (normalise, then gate)."""
    x, z = x.to(dtype), z.to(dtype)
    y = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps)
    if weight is not None:
        y = y * weight.to(dtype)
    return y * (z * torch.sigmoid(z))


def causal_conv1d_silu(x, w, cu_seqlens=None, dtype=torch.float64):
    """Depthwise causal conv over time, taps w [C, Kw] (tap Kw-1 multiplies x_t), zero history
    at each sequence start, then SiLU.  x [B, T, C]."""
    B, T, C = x.shape
    Kw = w.shape[1]
    x, w = x.to(dtype), w.to(dtype)
    y = torch.zeros_like(x)
    for (b, t0, t1) in _seq_bounds(B, T, cu_seqlens):
        xs = x[b, t0:t1]
        acc = torch.zeros_like(xs)
        for j in range(Kw):
            sh = Kw - 1 - j
            if sh == 0:
                acc += xs * w[:, j]
            elif sh < xs.shape[0]:
                acc[sh:] += xs[:-sh] * w[:, j]
        y[b, t0:t1] = acc * torch.sigmoid(acc)
    return y


def gate_beta(a, b, A_log, dt_bias, dtype=torch.float64):
    """g = -exp(A_log) * softplus(a + dt_bias);  beta = sigmoid(b)."""
    a, b, A_log, dt_bias = (t.to(dtype) for t in (a, b, A_log, dt_bias))
    return -torch.exp(A_log) * F.softplus(a + dt_bias), torch.sigmoid(b)


def gdn_block_ref(x, w_in, conv_w, A_log, dt_bias, norm_weight, *, Hk, Hv, dk, dv, cu_seqlens=None,
                  round_bf16=True, dtype=torch.float64):
    """Whole block on the CPU: in-projection [q | k | v | z | b | a] -> causal conv1d + SiLU on q/k/v -> q/k L2 norm ->
    gate/beta -> token recurrence -> gated RMSNorm.  With ``round_bf16`` the projection and convolution outputs are
    rounded to bf16 where the device pipeline stores them as bf16, so the comparison isolates kernel error."""
    B, T, hidden = x.shape
    rb = (lambda t: t.to(torch.bfloat16).to(dtype)) if round_bf16 else (lambda t: t)
    y = rb(x.to(dtype) @ w_in.to(dtype).T)
    nq = nk = Hk * dk
    nv = Hv * dv
    qkv = rb(causal_conv1d_silu(y[..., : nq + nk + nv], conv_w, cu_seqlens, dtype=dtype))
    z = y[..., nq + nk + nv: nq + nk + 2 * nv].reshape(B, T, Hv, dv)
    b_in = y[..., nq + nk + 2 * nv: nq + nk + 2 * nv + Hv]
    a_in = y[..., nq + nk + 2 * nv + Hv: nq + nk + 2 * nv + 2 * Hv]
    q = l2norm(qkv[..., :nq].reshape(B, T, Hk, dk))
    k = l2norm(qkv[..., nq: nq + nk].reshape(B, T, Hk, dk))
    v = qkv[..., nq + nk:].reshape(B, T, Hv, dv)
    g, beta = gate_beta(a_in, b_in, A_log, dt_bias, dtype=dtype)
    g, beta = g.float().to(dtype), beta.float().to(dtype)  # the device stores g and beta in fp32
    o, _ = naive_recurrent_gated_delta_rule(q, k, v, g, beta, dk ** -0.5, None, cu_seqlens, dtype=dtype)
    return gated_rmsnorm(o, z, norm_weight, dtype=dtype)


def rel_l2(x: torch.Tensor, ref: torch.Tensor) -> float:
    x, ref = x.double(), ref.double()
    den = ref.norm().item()
    return (x - ref).norm().item() / (den if den > 0 else 1.0)


def recurrent_grads(q, k, v, g, beta, d_o, scale=None, initial_state=None, d_final_state=None, cu_seqlens=None):
    """Gradients of the token recurrence by automatic differentiation of ``naive_recurrent_gated_delta_rule`` in fp64:
    returns (dq, dk, dv, dg, dbeta, d_initial_state or None) for the cotangents ``d_o`` (of o) and ``d_final_state``."""
    leaves = [t.detach().double().requires_grad_(True) for t in (q, k, v, g, beta)]
    s0 = initial_state.detach().double().requires_grad_(True) if initial_state is not None else None
    o, final = naive_recurrent_gated_delta_rule(*leaves, scale, s0, cu_seqlens)
    loss = (o * d_o.double()).sum()
    if d_final_state is not None:
        loss = loss + (final * d_final_state.double()).sum()
    grads = torch.autograd.grad(loss, leaves + ([s0] if s0 is not None else []))
    return (*grads[:5], grads[5] if s0 is not None else None)
