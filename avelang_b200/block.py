"""Qwen3-Next gated-delta-net block, sharded by heads across the GPUs of one node.

Order of operations: bf16 in-projection (this rank's columns only) -> depthwise causal conv1d (kernel 4) + SiLU on
q/k/v -> q/k L2 norm (inside the delta-rule kernel) -> gate/beta -> chunked delta rule on this rank's heads ->
gated RMSNorm (fused into the delta-rule epilogue) -> all-gather of the per-head outputs over NCCL.

Partitioning: rank r of G owns key heads [r*Hk/G, (r+1)*Hk/G) and the value heads that read them.  Every
(sequence, value head) recurrence is independent, so nothing crosses GPUs before the final all-gather; the
in-projection weight is sliced by output column so that each rank produces exactly its own heads.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class HeadShard:
    """Head ranges of one rank."""
    rank: int
    world: int
    Hk: int
    Hv: int

    def __post_init__(self):
        if self.Hk % self.world or self.Hv % self.Hk:
            raise ValueError(f"key heads ({self.Hk}) must divide by the world size ({self.world}) and value heads "
                             f"({self.Hv}) by key heads")

    @property
    def key_heads(self) -> range:
        n = self.Hk // self.world
        return range(self.rank * n, (self.rank + 1) * n)

    @property
    def value_heads(self) -> range:
        n = self.Hv // self.world
        return range(self.rank * n, (self.rank + 1) * n)


def projection_rows(shard: HeadShard, dk: int, dv: int) -> torch.Tensor:
    """Row indices of the fused in-projection weight [q | k | v | z | b | a] (rows = output features) that produce
    this rank's heads, in the order q, k, v, z, b, a."""
    Hk, Hv = shard.Hk, shard.Hv
    off_q, off_k, off_v = 0, Hk * dk, 2 * Hk * dk
    off_z, off_b, off_a = off_v + Hv * dv, off_v + 2 * Hv * dv, off_v + 2 * Hv * dv + Hv
    kh, vh = shard.key_heads, shard.value_heads
    parts = [torch.arange(off_q + kh.start * dk, off_q + kh.stop * dk),
             torch.arange(off_k + kh.start * dk, off_k + kh.stop * dk),
             torch.arange(off_v + vh.start * dv, off_v + vh.stop * dv),
             torch.arange(off_z + vh.start * dv, off_z + vh.stop * dv),
             torch.arange(off_b + vh.start, off_b + vh.stop),
             torch.arange(off_a + vh.start, off_a + vh.stop)]
    return torch.cat(parts)


def pad_rows(n: int, multiple: int = 8) -> int:
    return (n + multiple - 1) // multiple * multiple


class GdnBlockShard:
    """One rank's slice of the block.  ``w_in`` is the full fused projection weight ``[2*Hk*dk + 2*Hv*dv + 2*Hv, hidden]``;
    ``conv_w`` the full depthwise filter ``[2*Hk*dk + Hv*dv, 4]``; ``A_log``, ``dt_bias``, ``norm_weight`` per value head /
    per feature.  Only this rank's rows are kept on the device."""

    def __init__(self, w_in, conv_w, A_log, dt_bias, norm_weight, *, Hk, Hv, dk, dv, rank=0, world=1, device="cuda"):
        self.shard = HeadShard(rank, world, Hk, Hv)
        self.Hk, self.Hv, self.dk, self.dv = Hk, Hv, dk, dv
        self.hk_local, self.hv_local = Hk // world, Hv // world
        rows = projection_rows(self.shard, dk, dv)
        self.n_rows = rows.numel()
        w = w_in[rows].to(torch.bfloat16)
        pad = pad_rows(self.n_rows) - self.n_rows
        if pad:
            w = torch.cat([w, torch.zeros(pad, w.shape[1], dtype=w.dtype)], 0)
        self.w = w.to(device).contiguous()
        nq, nk, nv = self.hk_local * dk, self.hk_local * dk, self.hv_local * dv
        self.splits = (nq, nk, nv, nv, self.hv_local, self.hv_local)
        conv_rows = rows[: nq + nk + nv].clone()
        # conv filter rows follow the q | k | v feature order of the projection
        self.conv_w = conv_w[conv_rows].to(torch.bfloat16).to(device).contiguous()
        vh = self.shard.value_heads
        self.A_log = A_log[vh.start:vh.stop].float().to(device).contiguous()
        self.dt_bias = dt_bias[vh.start:vh.stop].float().to(device).contiguous()
        self.norm_weight = None if norm_weight is None else norm_weight.float().to(device).contiguous()

    def forward_local(self, x: torch.Tensor, cu_seqlens=None, out=None, out_peers=None, keep: dict | None = None) -> torch.Tensor:
        """x: bf16 [B, T, hidden] (replicated on every rank).  Returns this rank's normalised head outputs
        [B, T, Hv/G, dv] (written into ``out`` / scattered to ``out_peers`` when given).  ``keep``: a dict that receives
        the delta-rule stage's own inputs (q, k, v after the convolution, g, beta, z), so that a test can hold that
        stage alone against the checker."""
        from . import gdn, gemm
        B, T, hidden = x.shape
        y2 = gemm.gemm_pipeline_transposed_b(x.reshape(B * T, hidden), self.w)
        y = y2.reshape(B, T, -1)
        nq, nk, nv, nz, nb, na = self.splits
        qkv_in = y[:, :, : nq + nk + nv]
        z = y[:, :, nq + nk + nv: nq + nk + nv + nz].reshape(B, T, self.hv_local, self.dv)
        o0 = nq + nk + nv + nz
        b_in, a_in = y2[:, o0: o0 + nb], y2[:, o0 + nb: o0 + nb + na]
        qkv = gdn.causal_conv1d_silu(qkv_in, self.conv_w, cu_seqlens=cu_seqlens)
        q = qkv[:, :, :nq].reshape(B, T, self.hk_local, self.dk)
        k = qkv[:, :, nq: nq + nk].reshape(B, T, self.hk_local, self.dk)
        v = qkv[:, :, nq + nk:].reshape(B, T, self.hv_local, self.dv)
        g, beta = gdn.gate_beta(a_in, b_in, self.A_log, self.dt_bias)
        g, beta = g.reshape(B, T, self.hv_local), beta.reshape(B, T, self.hv_local)
        if keep is not None:
            keep.update(q=q, k=k, v=v, g=g, beta=beta, z=z)
        o, _ = gdn.chunk_gated_delta_rule(q, k, v, g, beta, use_qk_l2norm_in_kernel=True, cu_seqlens=cu_seqlens,
                                          z=z, norm_weight=self.norm_weight, out=out, out_peers=out_peers)
        return o

    def forward(self, x: torch.Tensor, cu_seqlens=None, group=None, fused_gather=False) -> torch.Tensor:
        """Full block output [B, T, Hv, dv] on every rank.  Default: local heads, then an NCCL all-gather over the head
        dimension.  ``fused_gather=True``: the gated-norm kernel stores each normalised row straight into every rank's
        output buffer (symmetric memory, plain peer stores over NVLink), bracketed by two barriers."""
        if not fused_gather or self.shard.world == 1:
            return gather_heads(self.forward_local(x, cu_seqlens), self.shard.world, group)
        import torch.distributed as dist
        B, T, _ = x.shape
        full, peers = self._symmetric_output(B, T, x.device, group)
        hl = self.hv_local
        mine = full[:, :, self.shard.rank * hl:(self.shard.rank + 1) * hl]
        self._stream_barrier(group)   # every rank is done reading the previous contents of the buffers
        self.forward_local(x, cu_seqlens, out=mine, out_peers=peers)
        self._stream_barrier(group)   # every rank's stores have landed
        return full

    def _stream_barrier(self, group=None):
        """Cross-rank barrier in stream order: a one-element all-reduce on the current stream.  What follows it on this
        rank's stream runs after everything every rank enqueued before its own call; unlike ``dist.barrier`` the host
        does not wait, so the launches on either side stay queued back to back."""
        import torch.distributed as dist
        tok = self.__dict__.get("_barrier_token")
        if tok is None:
            tok = self.__dict__["_barrier_token"] = torch.zeros(1, dtype=torch.int32, device=self.w.device)
        dist.all_reduce(tok, group=group)

    def _symmetric_output(self, B, T, device, group):
        """Output buffer [B, T, Hv, dv] in symmetric memory plus the device array of every rank's base address for this
        rank's head slice; cached per shape."""
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        key = (B, T, str(device))
        cache = self.__dict__.setdefault("_symm_cache", {})
        if key not in cache:
            grp = group if group is not None else dist.group.WORLD
            full = symm.empty((B, T, self.Hv, self.dv), dtype=torch.bfloat16, device=device)
            handle = symm.rendezvous(full, grp)
            off = self.shard.rank * self.hv_local * self.dv * full.element_size()
            peers = torch.tensor([int(p) + off for p in handle.buffer_ptrs], dtype=torch.int64, device=device)
            cache[key] = (full, peers, handle)
        full, peers, _ = cache[key]
        return full, peers


def output_projection_columns(shard: "HeadShard", dv: int) -> slice:
    """Columns of the output-projection weight ``[hidden, Hv*dv]`` that multiply this shard's value heads."""
    vh = shard.value_heads
    return slice(vh.start * dv, vh.stop * dv)


class GdnBlockTP(GdnBlockShard):
    """Tensor-parallel form of the block with the output projection: each rank multiplies its own heads' normalised
    output by its column slice of ``w_out [hidden, Hv*dv]`` (row-parallel linear) and the partial results are summed
    with one all-reduce, so no all-gather of head outputs is needed."""

    def __init__(self, w_in, conv_w, A_log, dt_bias, norm_weight, w_out, *, Hk, Hv, dk, dv, rank=0, world=1, device="cuda"):
        super().__init__(w_in, conv_w, A_log, dt_bias, norm_weight, Hk=Hk, Hv=Hv, dk=dk, dv=dv, rank=rank, world=world,
                         device=device)
        cols = output_projection_columns(self.shard, dv)
        self.w_out = w_out[:, cols].to(torch.bfloat16).to(device).contiguous()  # [hidden, hl*dv]

    def forward(self, x: torch.Tensor, cu_seqlens=None, group=None, fused_reduce=False) -> torch.Tensor:
        """Returns the block output after the output projection, ``[B, T, hidden]`` bf16, identical on every rank."""
        B, T, _ = x.shape
        o = self.forward_local(x, cu_seqlens)                                   # [B, T, hl, dv]
        return self.project(o.reshape(B * T, -1), group, fused_reduce).reshape(B, T, -1)

    def project(self, o2d: torch.Tensor, group=None, fused_reduce=False) -> torch.Tensor:
        """Output projection of this rank's normalised head outputs ``[M, hl*dv]`` and the sum over ranks, ``[M, hidden]``.
        Default: this rank's partial product, then one NCCL all-reduce.  ``fused_reduce=True``: the GEMM's epilogue stores
        each row of the partial product into the staging buffer of the rank that owns the row (symmetric memory, plain
        peer stores over NVLink, under the next tile's main loop); after a barrier every owner sums its rows in fp32 and
        stores them into every rank's result; a last barrier.  The fused result lives in a cached symmetric buffer that
        the next fused call overwrites."""
        from . import gemm
        if not fused_reduce or self.shard.world == 1:
            part = gemm.gemm_pipeline_transposed_b(o2d, self.w_out)              # this rank's partial sum
            if self.shard.world > 1:
                import torch.distributed as dist
                dist.all_reduce(part, group=group)
            return part
        stage, stage_peers, out, out_peers = self._symmetric_projection(o2d.shape[0], o2d.device, group)
        self._stream_barrier(group)   # every rank has consumed the previous result and its staging slots
        gemm.gemm_scatter_to_owners(o2d, self.w_out, stage, stage_peers, self.shard.rank)
        self._stream_barrier(group)   # every rank's partial rows have landed at their owners
        gemm.reduce_push_to_all(stage, out_peers, out, self.shard.rank)
        self._stream_barrier(group)   # every owner's rows have landed everywhere
        return out

    def _symmetric_projection(self, M, device, group):
        """Staging buffer [world, rows_per_owner, hidden] and result [M, hidden] in symmetric memory, with the device
        arrays of every rank's addresses; cached per M."""
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        key = ("proj", M, str(device))
        cache = self.__dict__.setdefault("_symm_cache", {})
        if key not in cache:
            grp = group if group is not None else dist.group.WORLD
            world, hidden = self.shard.world, self.w_out.shape[0]
            rpo = (M + world - 1) // world
            stage = symm.empty((world, rpo, hidden), dtype=torch.bfloat16, device=device)
            h1 = symm.rendezvous(stage, grp)
            out = symm.empty((M, hidden), dtype=torch.bfloat16, device=device)
            h2 = symm.rendezvous(out, grp)
            sp = torch.tensor([int(p) for p in h1.buffer_ptrs], dtype=torch.int64, device=device)
            op = torch.tensor([int(p) for p in h2.buffer_ptrs], dtype=torch.int64, device=device)
            cache[key] = (stage, sp, out, op, h1, h2)
        stage, sp, out, op, _, _ = cache[key]
        return stage, sp, out, op


def gather_heads(o_local: torch.Tensor, world: int, group=None) -> torch.Tensor:
    """All-gather of [B, T, Hv/G, dv] head slices into [B, T, Hv, dv] (rank-major gather, then one transpose copy)."""
    if world == 1:
        return o_local
    import torch.distributed as dist
    B, T, hl, dv = o_local.shape
    buf = torch.empty((world, B, T, hl, dv), dtype=o_local.dtype, device=o_local.device)
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(buf, o_local.contiguous(), group=group)
    else:  # host-side backends (used by the CPU tests) only have the list form
        dist.all_gather(list(buf.unbind(0)), o_local.contiguous(), group=group)
    return buf.permute(1, 2, 0, 3, 4).reshape(B, T, world * hl, dv)
