"""Seeded synthetic inputs for the gated-delta-net (GDN) path.

The draws follow one fixed order from a single CPU ``torch.Generator`` so that
the checker and the CUDA kernels always see identical bits: q, k (L2-normalised
per head vector), v, A_log, a, dt_bias, beta, then the optional extras (z,
states, slot indices, lengths).  q/k/v/z are rounded to bf16 before anything
consumes them; g and beta stay fp32.

Gate recipe: ``g = -exp(A_log) * softplus(a + dt_bias)`` with
``A_log ~ U(0, ln 16)`` per head, ``a ~ N(0,1)`` per token-head,
``dt_bias ~ N(0, 0.1)`` per head; ``beta = sigmoid(N(0,1))``.
``gate_scale`` multiplies g: 1.0 is the specified distribution, 0.01 is the
slow-decay variant that keeps the inter-chunk state path numerically visible.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch


@dataclass
class GdnInputs:
    q: torch.Tensor            # [B, T, Hk, dk]
    k: torch.Tensor            # [B, T, Hk, dk]
    v: torch.Tensor            # [B, T, Hv, dv]
    g: torch.Tensor            # [B, T, Hv] fp32, log decay (<= 0)
    beta: torch.Tensor         # [B, T, Hv] fp32
    scale: float
    z: torch.Tensor | None = None              # [B, T, Hv, dv]
    initial_state: torch.Tensor | None = None  # [N, Hv, dk, dv] fp32
    cu_seqlens: torch.Tensor | None = None     # [N+1] int32
    state_pool: torch.Tensor | None = None     # [slots, Hv, dk, dv] fp32
    state_indices: torch.Tensor | None = None  # [N] int32
    extras: dict = field(default_factory=dict)

    def to(self, device):
        def mv(x):
            return x.to(device) if isinstance(x, torch.Tensor) else x
        return GdnInputs(**{f: mv(getattr(self, f)) for f in self.__dataclass_fields__})


def _l2n(x: torch.Tensor) -> torch.Tensor:
    return x / x.norm(dim=-1, keepdim=True).clamp_min(1e-12)


def make_inputs(B, T, Hk, Hv, dk, dv, *, seed=0, dtype=torch.bfloat16, with_z=False,
                n_states=0, state_std=0.02, gate_scale=1.0, l2norm=True) -> GdnInputs:
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn(B, T, Hk, dk, generator=gen)
    k = torch.randn(B, T, Hk, dk, generator=gen)
    if l2norm:
        q, k = _l2n(q), _l2n(k)
    v = torch.randn(B, T, Hv, dv, generator=gen)
    A_log = torch.rand(Hv, generator=gen) * math.log(16.0)
    a = torch.randn(B, T, Hv, generator=gen)
    dt_bias = 0.1 * torch.randn(Hv, generator=gen)
    g = -torch.exp(A_log) * torch.nn.functional.softplus(a + dt_bias) * gate_scale
    beta = torch.sigmoid(torch.randn(B, T, Hv, generator=gen))
    z = torch.randn(B, T, Hv, dv, generator=gen).to(dtype) if with_z else None
    s0 = state_std * torch.randn(n_states, Hv, dk, dv, generator=gen) if n_states else None
    return GdnInputs(q=q.to(dtype), k=k.to(dtype), v=v.to(dtype), g=g.float().contiguous(),
                     beta=beta.float().contiguous(), scale=dk ** -0.5, z=z, initial_state=s0,
                     extras={"A_log": A_log, "dt_bias": dt_bias, "gen": gen})


def config0(seed=0) -> GdnInputs:
    """B=1, T=256, 4 heads, d=64, fp32 inputs, zero initial state."""
    return make_inputs(1, 256, 4, 4, 64, 64, seed=seed, dtype=torch.float32)


def config1(seed=0, T=8192, Hk=16, Hv=32, gate_scale=1.0) -> GdnInputs:
    """One Qwen3-Next GDN layer prefill: B=1, 16 key / 32 value heads, d=128, bf16, with z."""
    return make_inputs(1, T, Hk, Hv, 128, 128, seed=seed, with_z=True, gate_scale=gate_scale)


def config2(seed=0, n_seqs=256, n_slots=512, Hk=16, Hv=32, d=128) -> GdnInputs:
    """Continuous-batch decode step over a slot pool of fp32 states."""
    inp = make_inputs(n_seqs, 1, Hk, Hv, d, d, seed=seed)
    gen = inp.extras["gen"]
    inp.state_pool = 0.02 * torch.randn(n_slots, Hv, d, d, generator=gen)
    inp.state_indices = torch.randperm(n_slots, generator=gen)[:n_seqs].to(torch.int32)
    return inp


def varlen_lengths(n_seqs=64, lo=128, hi=16384, total=262144, seed=0) -> list[int]:
    """Log-uniform lengths in [lo, hi], rescaled to sum exactly to ``total``."""
    gen = torch.Generator().manual_seed(seed + 1000003)
    u = torch.rand(n_seqs, generator=gen, dtype=torch.float64)
    raw = torch.exp(math.log(lo) + u * (math.log(hi) - math.log(lo)))
    lens = torch.clamp(torch.round(raw * (total / raw.sum())), lo, hi).long()
    # put the remainder on the longest sequences without leaving [lo, hi]
    diff = int(total - lens.sum())
    order = torch.argsort(lens, descending=True).tolist()
    i = 0
    while diff != 0 and i < 16 * n_seqs:
        j = order[i % n_seqs]
        room = (hi - int(lens[j])) if diff > 0 else (int(lens[j]) - lo)
        step = max(-room, min(room, diff)) if diff > 0 else -min(room, -diff)
        lens[j] += step
        diff -= step
        i += 1
    if diff != 0:
        raise ValueError("cannot realise the requested total length inside [lo, hi]")
    return [int(x) for x in lens]


def config3(seed=0, n_seqs=64, lo=128, hi=16384, total=262144, Hk=16, Hv=32, d=128,
            gate_scale=1.0) -> GdnInputs:
    """Varlen packed prefill with nonzero initial states."""
    lens = varlen_lengths(n_seqs, lo, hi, total, seed)
    inp = make_inputs(1, total, Hk, Hv, d, d, seed=seed, n_states=n_seqs, gate_scale=gate_scale)
    cu = torch.zeros(n_seqs + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(lens, dtype=torch.int64).cumsum(0).to(torch.int32)
    inp.cu_seqlens = cu
    inp.extras["lengths"] = lens
    return inp
