"""Gated-delta-net (GDN) linear attention for B200: chunked prefill, fused recurrent decode, gated RMSNorm.

Entry points follow the calling convention of the reference's kernel library
(python/avelang_kernels/amdgpu_gemm.py:458-494): plain module-level functions that take torch tensors,
raise ValueError on dtype/shape/device problems, allocate the result unless ``out=`` is given, enqueue on
torch's current stream of the tensors' device and return without synchronising.  The reference itself has
no GDN kernels; the numerical contract is the recurrence

    M <- exp(g_t) M;  r = M^T k_t;  u = beta_t (v_t - r);  M <- M + k_t u^T;  o_t = scale M^T q_t

with M the fp32 key-major state [dk, dv] of one (sequence, value head).

Layouts: q, k ``[B, T, Hk, dk]``; v, z, o ``[B, T, Hv, dv]``; g (log decay) and beta ``[B, T, Hv]`` fp32; value head
h reads key head ``h // (Hv // Hk)``.  Varlen: ``B == 1`` and int32 ``cu_seqlens [N+1]`` on the device.  States:
fp32 ``[N or num_slots, Hv, dk, dv]``.  The innermost dimension must be contiguous; head/token/batch strides
are free as long as rows stay 16-byte aligned, so head-sharded slices of a packed tensor are accepted as is.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib, torch_ops

__all__ = ["chunk_gated_delta_rule", "fused_recurrent_gated_delta_rule", "mixed_prefill_decode_step", "gated_rmsnorm",
           "causal_conv1d_silu", "causal_conv1d_update", "gate_beta", "decode_layer_step", "gated_delta_rule_backward", "GatedDeltaRuleFunction", "prefill_launch_count", "read_status"]

_status_words: dict[int, torch.Tensor] = {}
_workspaces: dict[tuple[int, int], torch.Tensor] = {}


def _status_word(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _status_words:
        _status_words[idx] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status_words[idx]


def read_status(device=None, reset: bool = True) -> int:
    """Device status word accumulated by earlier calls (synchronises).  Bits: 1 = a state index beyond the
    pool, 2 = malformed cu_seqlens, 4 = a bounded device wait gave up.  The affected sequences were skipped."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    w = _status_word(device)
    val = int(w.item())
    if reset and val:
        w.zero_()
    return val


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Scratch owned by the Python layer, grown on demand and reused (one per device and stream)."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    cur = _workspaces.get(key)
    if cur is None or cur.numel() < nbytes:
        cur = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=device)
        _workspaces[key] = cur
    return cur


def _req(cond: bool, msg: str) -> None:
    if not cond:
        raise ValueError(msg)


def _check_common(q, k, v, g, beta, z, cu_seqlens):
    for name, t in (("q", q), ("k", k), ("v", v)):
        _req(isinstance(t, torch.Tensor) and t.dim() == 4, f"{name} must be a 4-D tensor [B, T, H, d]")
        _req(t.dtype == torch.bfloat16, f"{name} must have dtype torch.bfloat16, got {t.dtype}.")
        _req(t.is_cuda, f"{name} must be a CUDA tensor")
        _req(t.stride(-1) == 1, f"{name} must be contiguous in its last dimension")
        _req(t.device == q.device, f"{name} must be on device {q.device}, got {t.device}.")
    B, T, Hk, dk = q.shape
    _req(k.shape == q.shape, f"k must have shape {tuple(q.shape)}, got {tuple(k.shape)}.")
    _req(v.shape[0] == B and v.shape[1] == T, f"v must have leading shape {(B, T)}, got {tuple(v.shape[:2])}.")
    Hv, dv = v.shape[2], v.shape[3]
    _req(Hv % Hk == 0, f"value heads ({Hv}) must be a multiple of key heads ({Hk}).")
    _req((dk, dv) in ((128, 128), (64, 64)), f"head dims (dk, dv) must be (128, 128) or (64, 64), got {(dk, dv)}.")
    for name, t in (("g", g), ("beta", beta)):
        _req(t.dtype == torch.float32, f"{name} must have dtype torch.float32, got {t.dtype}.")
        _req(tuple(t.shape) == (B, T, Hv), f"{name} must have shape {(B, T, Hv)}, got {tuple(t.shape)}.")
        _req(t.device == q.device, f"{name} must be on device {q.device}, got {t.device}.")
        _req(t.stride(-1) == 1 or Hv == 1, f"{name} must be contiguous in its last dimension")
    _req(g.stride() == beta.stride(), "g and beta must share strides")
    if z is not None:
        _req(z.dtype == torch.bfloat16 and z.shape == v.shape and z.device == q.device and z.stride(-1) == 1,
             f"z must be a bf16 tensor of shape {tuple(v.shape)} on {q.device}")
    n_seqs = B
    if cu_seqlens is not None:
        _req(B == 1, "cu_seqlens requires B == 1 (packed layout)")
        _req(cu_seqlens.dtype == torch.int32 and cu_seqlens.dim() == 1 and cu_seqlens.numel() >= 1,
             "cu_seqlens must be a 1-D int32 tensor [N+1]")
        _req(cu_seqlens.device == q.device and cu_seqlens.is_contiguous(), f"cu_seqlens must be contiguous on {q.device}")
        n_seqs = cu_seqlens.numel() - 1
    return B, T, Hk, Hv, dk, dv, n_seqs


def _fill_args(q, k, v, g, beta, z, norm_weight, norm_eps, o, scale, initial_state, final_state, cu_seqlens,
               state_indices, num_slots, n_seqs, flags):
    B, T, Hk, dk = q.shape
    Hv, dv = v.shape[2], v.shape[3]
    a = _lib.GdnArgs()
    a.struct_size = ctypes.sizeof(_lib.GdnArgs)
    a.flags = flags
    ptr = lambda t: t.data_ptr() if t is not None and t.numel() > 0 else None
    a.q, a.k, a.v, a.g, a.beta, a.z, a.o = ptr(q), ptr(k), ptr(v), ptr(g), ptr(beta), ptr(z), ptr(o)
    a.norm_weight = ptr(norm_weight)
    a.initial_state, a.final_state = ptr(initial_state), ptr(final_state)
    a.cu_seqlens, a.state_indices = ptr(cu_seqlens), ptr(state_indices)
    a.status = _status_word(q.device).data_ptr()
    a.B, a.T, a.Hk, a.Hv, a.dk, a.dv = B, T, Hk, Hv, dk, dv
    a.n_seqs, a.num_slots, a.chunk = n_seqs, num_slots, 64
    for name, t in (("q", q), ("k", k), ("v", v), ("z", z), ("o", o)):
        if t is not None:
            setattr(a, f"{name}_stride_b", t.stride(0))
            setattr(a, f"{name}_stride_t", t.stride(1))
            setattr(a, f"{name}_stride_h", t.stride(2))
    a.g_stride_b, a.g_stride_t = g.stride(0), g.stride(1)
    a.scale = float(scale)
    a.norm_eps = float(norm_eps)
    return a


def _prep_out(out, v, z):
    if out is None:
        return torch.empty(v.shape, dtype=torch.bfloat16, device=v.device)
    _req(out.shape == v.shape, f"out must have shape {tuple(v.shape)}, got {tuple(out.shape)}.")
    _req(out.dtype == torch.bfloat16, f"out must have dtype torch.bfloat16, got {out.dtype}.")
    _req(out.device == v.device, f"out must be on device {v.device}, got {out.device}.")
    _req(out.stride(-1) == 1, "out must be contiguous in its last dimension")
    return out


def _prep_norm_weight(norm_weight, z, dv, device):
    if norm_weight is None:
        return None
    _req(z is not None, "norm_weight needs z (the gate of the fused RMSNorm)")
    _req(norm_weight.numel() == dv and norm_weight.device == device, f"norm_weight must have {dv} elements on {device}")
    return norm_weight.detach().float().contiguous()


def _prep_states(initial_state, state_indices, n_seqs, Hv, dk, dv, device, want_final, inplace):
    num_slots = n_seqs
    if initial_state is not None:
        _req(initial_state.dtype == torch.float32, f"initial_state must have dtype torch.float32, got {initial_state.dtype}.")
        _req(initial_state.dim() == 4 and tuple(initial_state.shape[1:]) == (Hv, dk, dv),
             f"initial_state must have shape [N, {Hv}, {dk}, {dv}], got {tuple(initial_state.shape)}.")
        _req(initial_state.is_contiguous() and initial_state.device == device, f"initial_state must be contiguous on {device}")
        num_slots = initial_state.shape[0]
    if state_indices is not None:
        _req(initial_state is not None, "state_indices needs initial_state (the state pool)")
        _req(state_indices.dtype == torch.int32 and tuple(state_indices.shape) == (n_seqs,),
             f"state_indices must be int32 of shape ({n_seqs},)")
        _req(state_indices.device == device and state_indices.is_contiguous(), f"state_indices must be contiguous on {device}")
    else:
        _req(initial_state is None or num_slots == n_seqs,
             f"initial_state must hold one state per sequence ({n_seqs}), got {num_slots}.")
    final = None
    if want_final:
        if state_indices is not None and inplace:
            final = initial_state
        elif state_indices is not None:
            final = initial_state.clone()
        else:
            final = torch.empty(n_seqs, Hv, dk, dv, dtype=torch.float32, device=device)
    return final, num_slots


def chunk_gated_delta_rule(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False,
                           use_qk_l2norm_in_kernel=False, cu_seqlens=None, *, z=None, norm_weight=None,
                           norm_eps=1e-6, state_indices=None, inplace_state=True, chunk_size=64, out=None, out_peers=None,
                           max_seqlen=None):
    """Chunked (chunk 64) gated delta rule over whole sequences.  Returns ``(o, final_state or None)``.

    With ``z`` the gated RMSNorm ``rmsnorm(o) * silu(z)`` (weight ``norm_weight``, eps ``norm_eps``) is fused and
    ``o`` is the normalised output.  With ``state_indices`` the initial states are read from, and the final
    states written to, slots of the ``initial_state`` pool (in place unless ``inplace_state=False``).

    ``out_peers`` (needs ``z``): int64 device tensor of base addresses of buffers laid out exactly like ``out``, one per
    GPU of the node (peer-mapped, this GPU's included).  The normalised rows are then stored into all of them by the
    norm kernel itself (a fused all-gather over NVLink) instead of into ``out``; the caller must put a barrier between
    this call and any reader of those buffers.

    ``max_seqlen`` (with ``cu_seqlens``): an upper bound of the longest sequence, known to the host.  With it the chunk
    ranges of the overlapped schedule (used for batches of few long sequences) are sized from the real chain length
    instead of the packed total; results are the same with or without it.  A sequence longer than the bound is skipped and flagged in the status word, like a
    malformed ``cu_seqlens`` entry."""
    B, T, Hk, Hv, dk, dv, n_seqs = _check_common(q, k, v, g, beta, z, cu_seqlens)
    _req(chunk_size == 64, f"chunk_size must be 64, got {chunk_size}.")
    _req(max_seqlen is None or int(max_seqlen) >= 0, f"max_seqlen must be non-negative, got {max_seqlen}.")
    o = _prep_out(out, v, z)
    norm_weight = _prep_norm_weight(norm_weight, z, dv, q.device)
    final, num_slots = _prep_states(initial_state, state_indices, n_seqs, Hv, dk, dv, q.device,
                                    output_final_state, inplace_state)
    if out_peers is not None:
        _req(z is not None, "out_peers needs z (the stores are fused into the gated norm)")
        _req(out_peers.dtype == torch.int64 and out_peers.dim() == 1 and out_peers.device == q.device and out_peers.is_contiguous(),
             f"out_peers must be a contiguous 1-D int64 tensor on {q.device}")
    bound = min(int(max_seqlen), T) if (max_seqlen is not None and cu_seqlens is not None) else 0
    torch_ops.op("chunk_prefill")(q, k, v, g, beta, o, float(dk ** -0.5 if scale is None else scale), initial_state, final,
                                  cu_seqlens, state_indices, z, norm_weight, float(norm_eps), bool(use_qk_l2norm_in_kernel),
                                  bound, out_peers)
    return o, final


@torch_ops.implement("chunk_prefill")
def _chunk_prefill(q, k, v, g, beta, out, scale, initial_state, final_state, cu_seqlens, state_indices, z, norm_weight,
                   norm_eps, qk_l2norm, max_seqlen, out_peers):
    """torch.ops.avelang_gdn.chunk_prefill: fills the C argument block and calls ave_gdn_chunk_prefill on the current
    stream, with scratch taken from the per-(device, stream) workspace this layer owns."""
    n_seqs = q.shape[0] if cu_seqlens is None else cu_seqlens.numel() - 1
    pool = final_state if final_state is not None else initial_state
    num_slots = pool.shape[0] if pool is not None else n_seqs
    a = _fill_args(q, k, v, g, beta, z, norm_weight, norm_eps, out, scale, initial_state, final_state, cu_seqlens,
                   state_indices, num_slots, n_seqs, _lib.FLAG_QK_L2NORM if qk_l2norm else 0)
    a.max_seqlen = int(max_seqlen)
    if out_peers is not None:
        a.o_peers, a.n_peers = out_peers.data_ptr(), out_peers.numel()
    lib = _lib.load()
    with torch.cuda.device(q.device):
        nbytes = lib.ave_gdn_prefill_workspace_bytes(ctypes.byref(a))
        ws = _workspace(q.device, nbytes)
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        rc = lib.ave_gdn_chunk_prefill(ctypes.byref(a), torch.cuda.current_stream(q.device).cuda_stream)
    _lib.check(rc, "chunk_gated_delta_rule")


def prefill_launch_count(q, k, v, *, z=None, cu_seqlens=None, max_seqlen=None, push=False) -> int:
    """Number of kernels one ``chunk_gated_delta_rule`` call on tensors of these shapes enqueues (``push``: with the
    fused all-gather).  Asked from the library, which derives it from the same schedule it launches."""
    B, T, Hk, dk = q.shape
    Hv, dv = v.shape[2], v.shape[3]
    n_seqs = B if cu_seqlens is None else cu_seqlens.numel() - 1
    a = _lib.GdnArgs()
    a.struct_size = ctypes.sizeof(_lib.GdnArgs)
    # only shapes, strides and the presence of optional tensors enter the count: nothing is read through the pointers
    a.q, a.k, a.v, a.o = q.data_ptr(), k.data_ptr(), v.data_ptr(), v.data_ptr()
    a.g = a.beta = v.data_ptr()
    a.z = z.data_ptr() if z is not None else None
    a.cu_seqlens = cu_seqlens.data_ptr() if cu_seqlens is not None else None
    a.B, a.T, a.Hk, a.Hv, a.dk, a.dv, a.n_seqs, a.num_slots, a.chunk = B, T, Hk, Hv, dk, dv, n_seqs, n_seqs, 64
    for name, t in (("q", q), ("k", k), ("v", v), ("z", z), ("o", v)):
        if t is not None:
            setattr(a, f"{name}_stride_b", t.stride(0)); setattr(a, f"{name}_stride_t", t.stride(1)); setattr(a, f"{name}_stride_h", t.stride(2))
    a.g_stride_b, a.g_stride_t = T * Hv, Hv
    if max_seqlen is not None and cu_seqlens is not None:
        a.max_seqlen = min(int(max_seqlen), T)
    if push:
        a.o_peers, a.n_peers = v.data_ptr(), 2  # only their presence matters for the count
    return int(_lib.load().ave_gdn_prefill_launch_count(ctypes.byref(a)))


def fused_recurrent_gated_delta_rule(q, k, v, g, beta, scale=None, initial_state=None, output_final_state=True,
                                     use_qk_l2norm_in_kernel=False, cu_seqlens=None, *, state_indices=None,
                                     inplace_state=True, z=None, norm_weight=None, norm_eps=1e-6, out=None):
    """Token-by-token gated delta rule with the state tile held on chip; ``T == 1`` with ``state_indices`` is the
    continuous-batching decode step: each sequence's state is streamed once in and once out of its slot of the
    ``initial_state`` pool (updated in place unless ``inplace_state=False``).  A negative slot index skips the
    sequence (no state access, zero output).  Returns ``(o, state)``."""
    B, T, Hk, Hv, dk, dv, n_seqs = _check_common(q, k, v, g, beta, z, cu_seqlens)
    o = _prep_out(out, v, z)
    norm_weight = _prep_norm_weight(norm_weight, z, dv, q.device)
    final, num_slots = _prep_states(initial_state, state_indices, n_seqs, Hv, dk, dv, q.device,
                                    output_final_state, inplace_state)
    torch_ops.op("decode_step")(q, k, v, g, beta, o, float(dk ** -0.5 if scale is None else scale), initial_state, final,
                                cu_seqlens, state_indices, z, norm_weight, float(norm_eps), bool(use_qk_l2norm_in_kernel))
    return o, final


@torch_ops.implement("decode_step")
def _decode_step(q, k, v, g, beta, out, scale, initial_state, final_state, cu_seqlens, state_indices, z, norm_weight,
                 norm_eps, qk_l2norm):
    """torch.ops.avelang_gdn.decode_step -> ave_gdn_decode_step on the current stream."""
    n_seqs = q.shape[0] if cu_seqlens is None else cu_seqlens.numel() - 1
    pool = final_state if final_state is not None else initial_state
    num_slots = pool.shape[0] if pool is not None else n_seqs
    a = _fill_args(q, k, v, g, beta, z, norm_weight, norm_eps, out, scale, initial_state, final_state, cu_seqlens,
                   state_indices, num_slots, n_seqs, _lib.FLAG_QK_L2NORM if qk_l2norm else 0)
    with torch.cuda.device(q.device):
        rc = _lib.load().ave_gdn_decode_step(ctypes.byref(a), torch.cuda.current_stream(q.device).cuda_stream)
    _lib.check(rc, "fused_recurrent_gated_delta_rule")


def mixed_prefill_decode_step(q, k, v, g, beta, cu_seqlens, n_decode, state_pool, state_indices, scale=None,
                              use_qk_l2norm_in_kernel=False, *, z=None, norm_weight=None, norm_eps=1e-6, out=None):
    """One continuous-batching step over a packed batch (``B == 1``) ordered decode-first: sequences ``[0, n_decode)``
    have exactly one token each and take the bandwidth-streaming decode kernel, the remaining sequences are prefill
    (or chunked-prefill continuation) sequences of any length and take the chunked kernel.  Every sequence reads its
    state from, and writes it back to, slot ``state_indices[n]`` of ``state_pool`` in place (a fresh sequence starts
    from a zeroed slot).  ``cu_seqlens`` describes the whole packed batch; its first ``n_decode + 1`` entries must be
    ``0, 1, ..., n_decode`` (not checked: that would need a device synchronisation).  Both launches go to the current
    stream.  Returns ``o`` ``[1, T, Hv, dv]``."""
    B, T, Hk, Hv, dk, dv, n_seqs = _check_common(q, k, v, g, beta, z, cu_seqlens)
    _req(cu_seqlens is not None and B == 1, "mixed_prefill_decode_step takes a packed batch: B == 1 with cu_seqlens")
    _req(0 <= n_decode <= n_seqs and n_decode <= T, f"n_decode must lie in [0, {min(n_seqs, T)}], got {n_decode}.")
    _req(state_pool is not None and state_indices is not None, "mixed_prefill_decode_step needs state_pool and state_indices")
    o = _prep_out(out, v, z)
    nd = int(n_decode)
    if nd > 0:
        step = lambda t: t[0, :nd].unsqueeze(1)  # [nd, 1, ...]: one single-token sequence per row
        fused_recurrent_gated_delta_rule(step(q), step(k), step(v), step(g), step(beta), scale, initial_state=state_pool,
                                         use_qk_l2norm_in_kernel=use_qk_l2norm_in_kernel, state_indices=state_indices[:nd].contiguous(),
                                         z=None if z is None else step(z), norm_weight=norm_weight, norm_eps=norm_eps, out=step(o))
    if nd < n_seqs:
        rest = lambda t: t[:, nd:]
        chunk_gated_delta_rule(rest(q), rest(k), rest(v), rest(g), rest(beta), scale, initial_state=state_pool,
                               output_final_state=True, use_qk_l2norm_in_kernel=use_qk_l2norm_in_kernel,
                               cu_seqlens=(cu_seqlens[nd:] - nd).contiguous(), z=None if z is None else rest(z),
                               norm_weight=norm_weight, norm_eps=norm_eps, state_indices=state_indices[nd:].contiguous(),
                               out=rest(o))
    return o


def gated_delta_rule_backward(q, k, v, g, beta, d_o, scale=None, initial_state=None, d_final_state=None, cu_seqlens=None):
    """Gradients of ``chunk_gated_delta_rule`` / ``fused_recurrent_gated_delta_rule`` (without the in-kernel L2 norm and
    without the fused gated norm) for d = 128.  ``d_o``: bf16, shaped like ``v``; ``d_final_state``: optional fp32 gradient
    of the final states.  Returns ``(dq, dk, dv, dg, dbeta, d_initial_state)``: dq, dk in the dtype and shape of q, k (the
    value heads sharing a key head are summed), dv in the dtype of v, dg, dbeta fp32, ``d_initial_state`` fp32 or None
    when no initial state was given.  A token-by-token reverse sweep in fp32 (recomputing the states from 64-token
    checkpoints): exact to fp32 rounding, and far slower than the chunked forward pass."""
    B, T, Hk, Hv, dk, dv, n_seqs = _check_common(q, k, v, g, beta, None, cu_seqlens)
    _req((dk, dv) == (128, 128), f"the backward pass is built for head dims (128, 128), got {(dk, dv)}.")
    _req(d_o.dtype == torch.bfloat16 and d_o.shape == v.shape and d_o.device == q.device and d_o.stride(-1) == 1,
         f"d_o must be a bf16 tensor of shape {tuple(v.shape)} on {q.device}")
    for name, t in (("initial_state", initial_state), ("d_final_state", d_final_state)):
        if t is not None:
            _req(t.dtype == torch.float32 and tuple(t.shape) == (n_seqs, Hv, dk, dv) and t.is_contiguous() and t.device == q.device,
                 f"{name} must be a contiguous fp32 tensor ({n_seqs}, {Hv}, {dk}, {dv}) on {q.device}")
    f32 = dict(dtype=torch.float32, device=q.device)
    dq_v, dk_v = torch.empty(B, T, Hv, dk, **f32), torch.empty(B, T, Hv, dk, **f32)
    dv_f, dg, dbeta = torch.empty(B, T, Hv, dv, **f32), torch.empty(B, T, Hv, **f32), torch.empty(B, T, Hv, **f32)
    ds0 = torch.empty(n_seqs, Hv, dk, dv, **f32) if initial_state is not None else None
    torch_ops.op("recurrent_backward")(q, k, v, g, beta, d_o, float(dk ** -0.5 if scale is None else scale), initial_state,
                                       d_final_state, cu_seqlens, dq_v, dk_v, dv_f, dg, dbeta, ds0)
    r = Hv // Hk
    dq = dq_v.view(B, T, Hk, r, dk).sum(3).to(q.dtype)
    dk_ = dk_v.view(B, T, Hk, r, dk).sum(3).to(k.dtype)
    return dq, dk_, dv_f.to(v.dtype), dg, dbeta, ds0


@torch_ops.implement("recurrent_backward")
def _recurrent_backward(q, k, v, g, beta, d_o, scale, initial_state, d_final_state, cu_seqlens, dq, dk, dv, dg, dbeta, d_initial_state):
    """torch.ops.avelang_gdn.recurrent_backward -> ave_gdn_recurrent_backward on the current stream."""
    B, T, Hk, dkk = q.shape
    Hv, dvv = v.shape[2], v.shape[3]
    a = _lib.BwdArgs()
    a.struct_size = ctypes.sizeof(_lib.BwdArgs)
    ptr = lambda t: t.data_ptr() if t is not None and t.numel() > 0 else None
    a.q, a.k, a.v, a.g, a.beta, a.d_o = ptr(q), ptr(k), ptr(v), ptr(g), ptr(beta), ptr(d_o)
    a.initial_state, a.d_final_state, a.cu_seqlens = ptr(initial_state), ptr(d_final_state), ptr(cu_seqlens)
    a.d_q, a.d_k, a.d_v, a.d_g, a.d_beta, a.d_initial_state = ptr(dq), ptr(dk), ptr(dv), ptr(dg), ptr(dbeta), ptr(d_initial_state)
    a.status = _status_word(q.device).data_ptr()
    a.B, a.T, a.Hk, a.Hv, a.dk, a.dv = B, T, Hk, Hv, dkk, dvv
    a.n_seqs = B if cu_seqlens is None else cu_seqlens.numel() - 1
    for name, t in (("q", q), ("k", k), ("v", v), ("do", d_o)):
        setattr(a, f"{name}_stride_b", t.stride(0)); setattr(a, f"{name}_stride_t", t.stride(1)); setattr(a, f"{name}_stride_h", t.stride(2))
    a.g_stride_b, a.g_stride_t, a.scale = g.stride(0), g.stride(1), float(scale)
    lib = _lib.load()
    with torch.cuda.device(q.device):
        ws = _workspace(q.device, lib.ave_gdn_backward_workspace_bytes(ctypes.byref(a)))
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        rc = lib.ave_gdn_recurrent_backward(ctypes.byref(a), torch.cuda.current_stream(q.device).cuda_stream)
    _lib.check(rc, "gated_delta_rule_backward")


class GatedDeltaRuleFunction(torch.autograd.Function):
    """``o, final_state = GatedDeltaRuleFunction.apply(q, k, v, g, beta, scale, initial_state)``: the chunked forward pass
    with the reverse-sweep backward pass attached (d = 128, dense batches, no in-kernel L2 norm, no fused gated norm)."""

    @staticmethod
    def forward(ctx, q, k, v, g, beta, scale, initial_state):
        o, final = chunk_gated_delta_rule(q, k, v, g, beta, scale, initial_state, output_final_state=True)
        ctx.save_for_backward(q, k, v, g, beta, initial_state if initial_state is not None else torch.empty(0, device=q.device))
        ctx.scale, ctx.has_state = scale, initial_state is not None
        return o, final

    @staticmethod
    def backward(ctx, d_o, d_final):
        q, k, v, g, beta, s0 = ctx.saved_tensors
        d_o = torch.zeros_like(v) if d_o is None else d_o.to(torch.bfloat16).contiguous()
        d_final = None if d_final is None else d_final.float().contiguous()
        dq, dk, dv, dg, dbeta, ds0 = gated_delta_rule_backward(q, k, v, g, beta, d_o, ctx.scale, s0 if ctx.has_state else None, d_final)
        return dq, dk, dv, dg, dbeta, None, ds0


def decode_layer_step(proj, conv_weight, conv_state, A_log, dt_bias, state_pool, state_indices=None, *, Hk, Hv, conv_bias=None,
                      norm_weight=None, norm_eps=1e-6, scale=None, gate_first=False, out=None):
    """One decode step of a whole GDN layer behind its in-projection, in one kernel.  ``proj``: bf16 ``[N, >= 2*Hk*128 +
    2*Hv*128 + 2*Hv]``, each row the new token's projection ``[q | k | v | z | b | a]`` (a column slice of a wider matrix
    is accepted); ``conv_weight`` bf16 ``[2*Hk*128 + Hv*128, W]`` (W in 2..4, rows in q | k | v order), ``conv_state`` bf16
    ``[slots, W-1, C]`` and ``state_pool`` fp32 ``[slots, Hv, 128, 128]`` share the slot index ``state_indices[n]`` (or n)
    and are updated in place; ``A_log``, ``dt_bias`` ``[Hv]``.  Computes conv update + SiLU, q/k L2 norm, gate and beta,
    the delta-rule update and the gated RMSNorm with z; the results are those of ``causal_conv1d_update`` + ``gate_beta`` +
    ``fused_recurrent_gated_delta_rule`` run one after the other.  Returns ``o [N, Hv, 128]``."""
    d = 128
    _req(proj.dtype == torch.bfloat16 and proj.dim() == 2 and proj.is_cuda and proj.stride(1) == 1, "proj must be a bf16 CUDA tensor [N, columns]")
    N = proj.shape[0]
    _req(Hk > 0 and Hv > 0 and Hv % Hk == 0, f"value heads ({Hv}) must be a multiple of key heads ({Hk}).")
    Cn, cols = 2 * Hk * d + Hv * d, 2 * Hk * d + 2 * Hv * d + 2 * Hv
    _req(proj.shape[1] >= cols, f"proj must have at least {cols} columns, got {proj.shape[1]}.")
    _req(conv_weight.dtype == torch.bfloat16 and conv_weight.dim() == 2 and conv_weight.shape[0] == Cn and 2 <= conv_weight.shape[1] <= 4
         and conv_weight.device == proj.device, f"conv_weight must be a bf16 tensor [{Cn}, W] with W in 2..4 on {proj.device}")
    W = conv_weight.shape[1]
    _req(conv_state.dtype == torch.bfloat16 and conv_state.dim() == 3 and tuple(conv_state.shape[1:]) == (W - 1, Cn)
         and conv_state.is_contiguous() and conv_state.device == proj.device,
         f"conv_state must be a contiguous bf16 tensor [slots, {W - 1}, {Cn}] on {proj.device}")
    _req(state_pool.dtype == torch.float32 and state_pool.dim() == 4 and tuple(state_pool.shape[1:]) == (Hv, d, d)
         and state_pool.is_contiguous() and state_pool.device == proj.device,
         f"state_pool must be a contiguous fp32 tensor [slots, {Hv}, {d}, {d}] on {proj.device}")
    _req(state_pool.shape[0] == conv_state.shape[0], "conv_state and state_pool must have the same number of slots")
    if state_indices is not None:
        _req(state_indices.dtype == torch.int32 and tuple(state_indices.shape) == (N,) and state_indices.device == proj.device
             and state_indices.is_contiguous(), f"state_indices must be a contiguous int32 tensor ({N},) on {proj.device}")
    else:
        _req(state_pool.shape[0] >= N, "the pools need one slot per sequence when state_indices is not given")
    A_log, dt_bias = A_log.detach().float().contiguous(), dt_bias.detach().float().contiguous()
    _req(A_log.numel() == Hv and dt_bias.numel() == Hv and A_log.device == proj.device, f"A_log and dt_bias must have {Hv} elements on {proj.device}")
    if norm_weight is not None:
        _req(norm_weight.numel() == d and norm_weight.device == proj.device, f"norm_weight must have {d} elements on {proj.device}")
        norm_weight = norm_weight.detach().float().contiguous()
    if conv_bias is not None:
        _req(conv_bias.dtype == torch.bfloat16 and conv_bias.numel() == Cn and conv_bias.device == proj.device, f"conv_bias must be bf16 [{Cn}]")
        conv_bias = conv_bias.contiguous()
    if out is None:
        out = torch.empty((N, Hv, d), dtype=torch.bfloat16, device=proj.device)
    _req(tuple(out.shape) == (N, Hv, d) and out.dtype == torch.bfloat16 and out.device == proj.device and out.stride(2) == 1
         and out.stride(1) == d, f"out must be a bf16 tensor ({N}, {Hv}, {d}) with contiguous rows on {proj.device}")
    torch_ops.op("decode_layer_step")(proj, conv_weight.contiguous(), conv_bias, conv_state, A_log, dt_bias, norm_weight, state_pool,
                                      state_indices, out, int(Hk), int(Hv), float(d ** -0.5 if scale is None else scale), float(norm_eps),
                                      bool(gate_first))
    return out


@torch_ops.implement("decode_layer_step")
def _decode_layer_step(proj, conv_w, conv_bias, conv_state, A_log, dt_bias, norm_weight, state_pool, state_indices, out, Hk, Hv,
                       scale, norm_eps, gate_first):
    """torch.ops.avelang_gdn.decode_layer_step -> ave_gdn_decode_layer_step on the current stream."""
    a = _lib.DecodeLayerArgs()
    a.struct_size = ctypes.sizeof(_lib.DecodeLayerArgs)
    a.flags = _lib.FLAG_GATE_FIRST if gate_first else 0
    ptr = lambda t: t.data_ptr() if t is not None else None
    a.proj, a.conv_w, a.conv_bias, a.conv_state = ptr(proj), ptr(conv_w), ptr(conv_bias), ptr(conv_state)
    a.A_log, a.dt_bias, a.norm_weight, a.state_pool = ptr(A_log), ptr(dt_bias), ptr(norm_weight), ptr(state_pool)
    a.state_indices, a.o, a.status = ptr(state_indices), ptr(out), _status_word(proj.device).data_ptr()
    a.n_seqs, a.Hk, a.Hv, a.dk, a.dv, a.width, a.num_slots = proj.shape[0], Hk, Hv, 128, 128, conv_w.shape[1], state_pool.shape[0]
    a.proj_stride, a.o_stride, a.scale, a.norm_eps = proj.stride(0), out.stride(0), scale, norm_eps
    with torch.cuda.device(proj.device):
        rc = _lib.load().ave_gdn_decode_layer_step(ctypes.byref(a), torch.cuda.current_stream(proj.device).cuda_stream)
    _lib.check(rc, "decode_layer_step")


def gated_rmsnorm(x, z, weight=None, eps=1e-6, *, gate_first=False, out=None):
    """``y = weight * x * rsqrt(mean(x^2) + eps) * silu(z)`` over the last dimension (64 or 128), bf16 in/out,
    fp32 math.  ``x``/``z``/``out``: ``[..., H, d]`` with a contiguous last dimension."""
    _req(x.dtype == torch.bfloat16, f"x must have dtype torch.bfloat16, got {x.dtype}.")
    _req(z.dtype == torch.bfloat16, f"z must have dtype torch.bfloat16, got {z.dtype}.")
    _req(x.is_cuda and z.device == x.device, f"z must be on device {x.device}, got {z.device}.")
    _req(z.shape == x.shape, f"z must have shape {tuple(x.shape)}, got {tuple(z.shape)}.")
    _req(x.dim() >= 2 and x.shape[-1] in (64, 128), f"last dimension must be 64 or 128, got {x.shape[-1]}.")
    d, H = x.shape[-1], x.shape[-2]
    if out is None:
        out = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
    _req(out.shape == x.shape and out.dtype == torch.bfloat16 and out.device == x.device,
         f"out must be a bf16 tensor of shape {tuple(x.shape)} on {x.device}")
    x3, z3, y3 = (t.reshape(-1, H, d) if t.dim() != 3 else t for t in (x, z, out))
    _req(y3.data_ptr() == out.data_ptr(), "out must be viewable as [rows, H, d] without a copy")
    for t in (x3, z3, y3):
        _req(t.stride(-1) == 1, "tensors must be contiguous in their last dimension")
    w = None
    if weight is not None:
        _req(weight.numel() == d and weight.device == x.device, f"weight must have {d} elements on {x.device}")
        w = weight.detach().float().contiguous()
    torch_ops.op("gated_rmsnorm")(x3, z3, w, float(eps), bool(gate_first), y3)
    return out


@torch_ops.implement("gated_rmsnorm")
def _gated_rmsnorm(x3, z3, weight, eps, gate_first, y3):
    """torch.ops.avelang_gdn.gated_rmsnorm -> ave_gdn_gated_rmsnorm; tensors are [rows, H, d] views."""
    a = _lib.NormArgs()
    a.struct_size = ctypes.sizeof(_lib.NormArgs)
    a.flags = _lib.FLAG_GATE_FIRST if gate_first else 0
    a.x, a.z, a.y = x3.data_ptr(), z3.data_ptr(), y3.data_ptr()
    a.weight = weight.data_ptr() if weight is not None else None
    a.rows, a.d, a.heads, a.eps = x3.shape[0] * x3.shape[1], x3.shape[2], x3.shape[1], float(eps)
    a.x_stride_t, a.x_stride_h = x3.stride(0), x3.stride(1)
    a.z_stride_t, a.z_stride_h = z3.stride(0), z3.stride(1)
    a.y_stride_t, a.y_stride_h = y3.stride(0), y3.stride(1)
    with torch.cuda.device(x3.device):
        rc = _lib.load().ave_gdn_gated_rmsnorm(ctypes.byref(a), torch.cuda.current_stream(x3.device).cuda_stream)
    _lib.check(rc, "gated_rmsnorm")


def causal_conv1d_silu(x, weight, bias=None, cu_seqlens=None, *, out=None):
    """Depthwise causal convolution over time followed by SiLU: ``y[t, c] = silu(bias[c] + sum_j weight[c, j] *
    x[t - (W-1) + j, c])`` with zero history at the start of every sequence.  ``x``: bf16 ``[B, T, C]`` (channel
    stride 1, row stride free, so a column slice of a wider projection output is accepted), ``weight``: bf16
    ``[C, W]`` with W in 2..4, optional ``bias`` bf16 ``[C]``, optional int32 ``cu_seqlens`` (``B == 1``)."""
    _req(x.dtype == torch.bfloat16 and x.dim() == 3 and x.is_cuda, "x must be a bf16 CUDA tensor [B, T, C]")
    _req(x.stride(2) == 1, "x must be contiguous in its last dimension")
    B, T, Cn = x.shape
    _req(weight.dtype == torch.bfloat16 and weight.dim() == 2 and weight.shape[0] == Cn and weight.device == x.device,
         f"weight must be a bf16 tensor [{Cn}, W] on {x.device}")
    W = weight.shape[1]
    _req(2 <= W <= 4, f"kernel width must be 2, 3 or 4, got {W}.")
    _req(Cn % 8 == 0, f"channels must be a multiple of 8, got {Cn}.")
    weight = weight.contiguous()
    if bias is not None:
        _req(bias.dtype == torch.bfloat16 and bias.numel() == Cn and bias.device == x.device, f"bias must be bf16 [{Cn}] on {x.device}")
        bias = bias.contiguous()
    if out is None:
        out = torch.empty((B, T, Cn), dtype=torch.bfloat16, device=x.device)
    _req(out.shape == x.shape and out.dtype == torch.bfloat16 and out.device == x.device and out.stride(2) == 1,
         f"out must be a bf16 tensor of shape {tuple(x.shape)} on {x.device}")
    _req(out.data_ptr() != x.data_ptr(), "out must not alias x (later tokens read earlier inputs)")
    if cu_seqlens is not None:
        _req(B == 1 and cu_seqlens.dtype == torch.int32 and cu_seqlens.device == x.device and cu_seqlens.is_contiguous(),
             "cu_seqlens must be a contiguous int32 tensor on the device of x, with B == 1")
    torch_ops.op("conv1d_silu")(x, weight, bias, cu_seqlens, out)
    return out


@torch_ops.implement("conv1d_silu")
def _conv1d_silu(x, weight, bias, cu_seqlens, out):
    """torch.ops.avelang_gdn.conv1d_silu -> ave_gdn_conv1d_silu."""
    B, T, Cn = x.shape
    a = _lib.ConvArgs()
    a.struct_size = ctypes.sizeof(_lib.ConvArgs)
    a.x, a.w, a.y = x.data_ptr(), weight.data_ptr(), out.data_ptr()
    a.bias = bias.data_ptr() if bias is not None else None
    a.B, a.T, a.C, a.width = B, T, Cn, weight.shape[1]
    if cu_seqlens is not None:
        a.cu_seqlens, a.n_seqs = cu_seqlens.data_ptr(), cu_seqlens.numel() - 1
    a.x_stride_b, a.x_stride_t, a.y_stride_b, a.y_stride_t = x.stride(0), x.stride(1), out.stride(0), out.stride(1)
    with torch.cuda.device(x.device):
        rc = _lib.load().ave_gdn_conv1d_silu(ctypes.byref(a), torch.cuda.current_stream(x.device).cuda_stream)
    _lib.check(rc, "causal_conv1d_silu")


def causal_conv1d_update(x, conv_state, weight, bias=None, state_indices=None, *, out=None):
    """Decode-time step of ``causal_conv1d_silu``: ``x`` bf16 ``[N, C]`` (one new token per sequence), ``conv_state`` bf16
    ``[slots, W-1, C]`` holding each sequence's last W-1 inputs (oldest first), updated in place; optional int32
    ``state_indices [N]`` selects the slots (negative: skip that sequence; beyond the pool: skip it and raise bit 1 of
    the status word).  Returns ``y [N, C]``."""
    _req(x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_cuda and x.stride(1) == 1, "x must be a bf16 CUDA tensor [N, C]")
    N, Cn = x.shape
    W = weight.shape[1]
    _req(weight.dtype == torch.bfloat16 and tuple(weight.shape) == (Cn, W) and weight.device == x.device and 2 <= W <= 4,
         f"weight must be a bf16 tensor [{Cn}, W] with W in 2..4 on {x.device}")
    _req(Cn % 8 == 0, f"channels must be a multiple of 8, got {Cn}.")
    _req(conv_state.dtype == torch.bfloat16 and conv_state.dim() == 3 and tuple(conv_state.shape[1:]) == (W - 1, Cn)
         and conv_state.is_contiguous() and conv_state.device == x.device,
         f"conv_state must be a contiguous bf16 tensor [slots, {W - 1}, {Cn}] on {x.device}")
    if state_indices is not None:
        _req(state_indices.dtype == torch.int32 and tuple(state_indices.shape) == (N,) and state_indices.device == x.device
             and state_indices.is_contiguous(), f"state_indices must be a contiguous int32 tensor ({N},) on {x.device}")
    else:
        _req(conv_state.shape[0] >= N, "conv_state needs one slot per sequence when state_indices is not given")
    weight = weight.contiguous()
    if out is None:
        out = torch.empty((N, Cn), dtype=torch.bfloat16, device=x.device)
    _req(out.shape == x.shape and out.dtype == torch.bfloat16 and out.device == x.device and out.stride(1) == 1,
         f"out must be a bf16 tensor of shape {tuple(x.shape)} on {x.device}")
    bias = bias.contiguous() if bias is not None else None
    torch_ops.op("conv1d_update")(x, conv_state, weight, bias, state_indices, out)
    return out


@torch_ops.implement("conv1d_update")
def _conv1d_update(x, conv_state, weight, bias, state_indices, out):
    """torch.ops.avelang_gdn.conv1d_update -> ave_gdn_conv1d_update (history updated in place)."""
    N, Cn = x.shape
    a = _lib.ConvUpdateArgs()
    a.struct_size = ctypes.sizeof(_lib.ConvUpdateArgs)
    a.x, a.w, a.y, a.conv_state = x.data_ptr(), weight.data_ptr(), out.data_ptr(), conv_state.data_ptr()
    a.bias = bias.data_ptr() if bias is not None else None
    a.state_indices = state_indices.data_ptr() if state_indices is not None else None
    a.n_seqs, a.C, a.width, a.num_slots = N, Cn, weight.shape[1], conv_state.shape[0]
    a.x_stride, a.y_stride = x.stride(0), out.stride(0)
    a.status = _status_word(x.device).data_ptr()
    with torch.cuda.device(x.device):
        rc = _lib.load().ave_gdn_conv1d_update(ctypes.byref(a), torch.cuda.current_stream(x.device).cuda_stream)
    _lib.check(rc, "causal_conv1d_update")


def gate_beta(a_in, b_in, A_log, dt_bias):
    """``g = -exp(A_log) * softplus(a + dt_bias)`` and ``beta = sigmoid(b)`` in fp32.  ``a_in``, ``b_in``: bf16
    ``[..., Hv]`` (last dimension contiguous, one common row stride); ``A_log``, ``dt_bias``: ``[Hv]``."""
    _req(a_in.dtype == torch.bfloat16 and b_in.dtype == torch.bfloat16 and a_in.is_cuda, "a and b must be bf16 CUDA tensors")
    _req(a_in.shape == b_in.shape and a_in.stride(-1) == 1 and b_in.stride(-1) == 1, "a and b must share a shape [..., Hv]")
    Hv = a_in.shape[-1]
    a2, b2 = a_in.reshape(-1, Hv) if a_in.dim() != 2 else a_in, b_in.reshape(-1, Hv) if b_in.dim() != 2 else b_in
    _req(a2.data_ptr() == a_in.data_ptr() and b2.data_ptr() == b_in.data_ptr(), "a and b must be viewable as [rows, Hv]")
    A_log, dt_bias = A_log.detach().float().contiguous(), dt_bias.detach().float().contiguous()
    _req(A_log.numel() == Hv and dt_bias.numel() == Hv and A_log.device == a_in.device, f"A_log and dt_bias must have {Hv} elements")
    g = torch.empty(a_in.shape, dtype=torch.float32, device=a_in.device)
    beta = torch.empty_like(g)
    torch_ops.op("gate_beta")(a2, b2, A_log, dt_bias, g, beta)
    return g, beta


@torch_ops.implement("gate_beta")
def _gate_beta(a2, b2, A_log, dt_bias, g, beta):
    """torch.ops.avelang_gdn.gate_beta -> ave_gdn_gate_beta; a2, b2 are [rows, Hv] views."""
    s = _lib.GateArgs()
    s.struct_size = ctypes.sizeof(_lib.GateArgs)
    s.a, s.b, s.A_log, s.dt_bias, s.g, s.beta = (a2.data_ptr(), b2.data_ptr(), A_log.data_ptr(), dt_bias.data_ptr(),
                                                 g.data_ptr(), beta.data_ptr())
    s.rows, s.Hv, s.a_stride_row, s.b_stride_row = a2.shape[0], a2.shape[1], a2.stride(0), b2.stride(0)
    with torch.cuda.device(a2.device):
        rc = _lib.load().ave_gdn_gate_beta(ctypes.byref(s), torch.cuda.current_stream(a2.device).cuda_stream)
    _lib.check(rc, "gate_beta")
