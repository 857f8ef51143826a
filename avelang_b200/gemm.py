"""bf16 GEMM ``C = A @ B.T`` on the B200 tensor cores (tcgen05 / TMEM / TMA).

Same name, operand convention and error behaviour as the reference's
``gemm_pipeline_transposed_b`` (python/avelang_kernels/amdgpu_gemm.py:458-494): ``A [M, K]`` and ``B [N, K]``
(the layout of ``nn.Linear.weight``) in bf16, fp32 accumulation, bf16 result, optional ``out=``.  The reference
requires M % 128 == N % 128 == K % 64 == 0; here only K % 8 == 0 and 16-byte aligned rows are required."""
from __future__ import annotations

import ctypes

import torch

from . import _lib, gdn, torch_ops

__all__ = ["gemm_pipeline_transposed_b"]


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
