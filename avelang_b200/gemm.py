"""bf16 GEMM ``C = A @ B.T`` on the B200 tensor cores (tcgen05 / TMEM / TMA).

Same name, operand convention and error behaviour as the reference's
``gemm_pipeline_transposed_b`` (python/avelang_kernels/amdgpu_gemm.py:458-494): ``A [M, K]`` and ``B [N, K]``
(the layout of ``nn.Linear.weight``) in bf16, fp32 accumulation, bf16 result, optional ``out=``.  The reference
requires M % 128 == N % 128 == K % 64 == 0; here only K % 8 == 0 and 16-byte aligned rows are required."""
from __future__ import annotations

import ctypes

import torch

from . import _lib, gdn, torch_ops

__all__ = ["gemm_pipeline_transposed_b", "gemm_scatter_to_owners", "reduce_push_to_all"]


def gemm_pipeline_transposed_b(A: torch.Tensor, B: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    if A.dtype != torch.bfloat16:
        raise ValueError(f"A must have dtype torch.bfloat16, got {A.dtype}.")
    if B.dtype != torch.bfloat16:
        raise ValueError(f"B must have dtype torch.bfloat16, got {B.dtype}.")
    if A.dim() != 2 or B.dim() != 2 or A.shape[1] != B.shape[1]:
        raise ValueError(f"A [M, K] and B [N, K] must share K, got {tuple(A.shape)} and {tuple(B.shape)}.")
    if not A.is_cuda or B.device != A.device:
        raise ValueError(f"A and B must be CUDA tensors on one device, got {A.device} and {B.device}.")
    m, k = A.shape
    n = B.shape[0]
    if k % 8 != 0 or k == 0:
        raise ValueError(f"K must be a positive multiple of 8, got {k}.")
    if A.stride(1) != 1 or B.stride(1) != 1:
        raise ValueError("A and B must be contiguous in their last dimension.")
    out_shape = (m, n)
    if out is None:
        out = torch.empty(out_shape, dtype=torch.bfloat16, device=A.device)
    elif out.shape != out_shape:
        raise ValueError(f"out must have shape {out_shape}, got {tuple(out.shape)}.")
    elif out.dtype != torch.bfloat16:
        raise ValueError(f"out must have dtype torch.bfloat16, got {out.dtype}.")
    elif out.device != A.device:
        raise ValueError(f"out must be on device {A.device}, got {out.device}.")
    elif out.stride(1) != 1:
        raise ValueError("out must be contiguous in its last dimension.")
    torch_ops.op("gemm_bf16_nt")(A, B, out)
    return out


@torch_ops.implement("gemm_bf16_nt")
def _gemm_bf16_nt(A, B, out):
    """torch.ops.avelang_gdn.gemm_bf16_nt -> ave_gemm_bf16_nt on the current stream."""
    a = _lib.GemmArgs()
    a.struct_size = ctypes.sizeof(_lib.GemmArgs)
    a.a, a.b, a.c = A.data_ptr(), B.data_ptr(), out.data_ptr()
    a.M, a.N, a.K = A.shape[0], B.shape[0], A.shape[1]
    a.lda, a.ldb, a.ldc = A.stride(0), B.stride(0), out.stride(0)
    a.status = gdn._status_word(A.device).data_ptr()  # gdn.read_status() also reports a GEMM that gave up a wait
    with torch.cuda.device(A.device):
        rc = _lib.load().ave_gemm_bf16_nt(ctypes.byref(a), torch.cuda.current_stream(A.device).cuda_stream)
    _lib.check(rc, "gemm_pipeline_transposed_b")


# ---------------------------------------------------------------- row-parallel linear with the cross-rank sum fused in
def _reduce_args(stage, stage_peers, out_peers, rank, M, N, ldc, rows_per_owner):
    r = _lib.GemmReduceArgs()
    r.struct_size = ctypes.sizeof(_lib.GemmReduceArgs)
    r.M, r.N, r.ldc = M, N, ldc
    r.stage = stage.data_ptr()
    r.stage_peers = (stage_peers if stage_peers is not None else out_peers).data_ptr()
    r.out_peers = (out_peers if out_peers is not None else stage_peers).data_ptr()
    r.n_ranks, r.rank, r.rows_per_owner = stage.shape[0], rank, rows_per_owner
    r.status = gdn._status_word(stage.device).data_ptr()
    return r


def gemm_scatter_to_owners(A: torch.Tensor, B: torch.Tensor, stage: torch.Tensor, stage_peers: torch.Tensor, rank: int) -> None:
    """First phase of a row-parallel linear layer: ``A [M, K_local] @ B [N, K_local].T`` with the GEMM's epilogue storing
    each row of the partial product into slot ``rank`` of the staging buffer of the rank that owns the row.

    ``stage [n_ranks, rows_per_owner, N]`` bf16 is this rank's own staging buffer, ``stage_peers`` an int64 device
    tensor of every rank's staging-buffer address (peer-reachable memory).  A cross-rank barrier must follow before
    :func:`reduce_push_to_all`."""
    if A.dtype != torch.bfloat16 or B.dtype != torch.bfloat16 or stage.dtype != torch.bfloat16:
        raise ValueError("A, B and stage must have dtype torch.bfloat16.")
    if A.dim() != 2 or B.dim() != 2 or A.shape[1] != B.shape[1]:
        raise ValueError(f"A [M, K] and B [N, K] must share K, got {tuple(A.shape)} and {tuple(B.shape)}.")
    if stage.dim() != 3 or stage.shape[2] != B.shape[0] or not stage.is_contiguous():
        raise ValueError(f"stage must be a contiguous [n_ranks, rows_per_owner, N={B.shape[0]}] tensor, got {tuple(stage.shape)}.")
    if stage.shape[0] * stage.shape[1] < A.shape[0]:
        raise ValueError(f"{stage.shape[0]} owners of {stage.shape[1]} rows cannot hold M={A.shape[0]} rows.")
    if stage_peers.dtype != torch.int64 or stage_peers.numel() != stage.shape[0]:
        raise ValueError("stage_peers must hold one int64 address per rank.")
    if A.shape[1] % 8 != 0 or A.shape[1] == 0 or A.stride(1) != 1 or B.stride(1) != 1:
        raise ValueError("K must be a positive multiple of 8 and A, B contiguous in their last dimension.")
    torch_ops.op("gemm_scatter")(A, B, stage, stage_peers, rank, stage.shape[1])


def reduce_push_to_all(stage: torch.Tensor, out_peers: torch.Tensor, out: torch.Tensor, rank: int) -> None:
    """Second phase: this rank sums its rows over the slots of its staging buffer (fp32, slot order, one rounding) and
    stores them into every rank's result matrix ``out [M, N]`` (``out_peers``: int64 device tensor of their addresses).
    A cross-rank barrier must follow before ``out`` is read."""
    if stage.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or out.dim() != 2 or out.stride(1) != 1:
        raise ValueError("stage and out must be bf16, out [M, N] contiguous in its last dimension.")
    if out_peers.dtype != torch.int64 or out_peers.numel() != stage.shape[0]:
        raise ValueError("out_peers must hold one int64 address per rank.")
    torch_ops.op("gemm_reduce_push")(stage, out_peers, out, rank, out.shape[0], stage.shape[1])


@torch_ops.implement("gemm_scatter")
def _gemm_scatter(A, B, stage, stage_peers, rank, rows_per_owner):
    """torch.ops.avelang_gdn.gemm_scatter -> ave_gemm_bf16_nt_scatter on the current stream."""
    r = _reduce_args(stage, stage_peers, None, rank, A.shape[0], B.shape[0], B.shape[0], rows_per_owner)
    r.a, r.b, r.K, r.lda, r.ldb = A.data_ptr(), B.data_ptr(), A.shape[1], A.stride(0), B.stride(0)
    with torch.cuda.device(A.device):
        rc = _lib.load().ave_gemm_bf16_nt_scatter(ctypes.byref(r), torch.cuda.current_stream(A.device).cuda_stream)
    _lib.check(rc, "gemm_scatter_to_owners")


@torch_ops.implement("gemm_reduce_push")
def _gemm_reduce_push(stage, out_peers, out, rank, M, rows_per_owner):
    """torch.ops.avelang_gdn.gemm_reduce_push -> ave_gemm_reduce_push on the current stream."""
    r = _reduce_args(stage, None, out_peers, rank, M, stage.shape[2], out.stride(0), rows_per_owner)
    with torch.cuda.device(stage.device):
        rc = _lib.load().ave_gemm_reduce_push(ctypes.byref(r), torch.cuda.current_stream(stage.device).cuda_stream)
    _lib.check(rc, "reduce_push_to_all")
