"""ctypes wrapper around the C checker (libgdn_oracle.so).  TEST INFRASTRUCTURE ONLY."""
from __future__ import annotations

import ctypes
import os
import subprocess

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build(force: bool = False) -> str:
    so = os.path.join(_HERE, "libgdn_oracle.so")
    src = os.path.join(_HERE, "gdn_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "libgdn_oracle.so"], check=True, capture_output=True)
    return so


def _lib():
    global _LIB
    if _LIB is None:
        _LIB = ctypes.CDLL(build())
    return _LIB


def set_threads(n: int) -> int:
    """Sets the OpenMP team size of the C routines (launchers such as torchrun export OMP_NUM_THREADS=1, which would
    otherwise pin the timed CPU baseline to one core).  Returns the count set, 0 if the OpenMP runtime was not found."""
    _lib()  # makes sure the runtime the library links against is loaded
    try:
        ctypes.CDLL("libgomp.so.1").omp_set_num_threads(int(n))
        return int(n)
    except OSError:
        return 0


def recurrent(q, k, v, g, beta, scale=None, initial_state=None, cu_seqlens=None, precision="f64",
              use_qk_l2norm_in_kernel=False):
    """Same function as gdn_oracle.naive_recurrent_gated_delta_rule, run by the C checker.
    Accepts [B,T,H,d] tensors (any float dtype; widened to fp32 exactly); returns fp32 (o, final_state)."""
    B, T, Hk, dk = q.shape
    Hv, dv = v.shape[-2], v.shape[-1]
    scale = dk ** -0.5 if scale is None else scale
    f = lambda x: x.detach().cpu().float().contiguous()
    q, k, v, g, beta = f(q), f(k), f(v), f(g), f(beta)
    if cu_seqlens is None:
        cu = torch.arange(0, (B + 1) * T, T, dtype=torch.int32)
    else:
        cu = cu_seqlens.detach().cpu().to(torch.int32).contiguous()
    N = cu.numel() - 1
    o = torch.zeros(B, T, Hv, dv, dtype=torch.float32)
    sT = torch.zeros(N, Hv, dk, dv, dtype=torch.float32)
    s0 = f(initial_state) if initial_state is not None else None
    fn = getattr(_lib(), "gdn_oracle_recurrent_" + precision)
    P, I64, I32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32
    fn.argtypes = [P] * 9 + [I32] * 5 + [I64] * 5 + [ctypes.c_float, I32]
    fn.restype = ctypes.c_int
    rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(),
            s0.data_ptr() if s0 is not None else None, o.data_ptr(), sT.data_ptr(), cu.data_ptr(),
            N, Hk, Hv, dk, dv, Hk * dk, Hk * dk, Hv * dv, Hv * dv, Hv, float(scale),
            int(use_qk_l2norm_in_kernel))
    if rc != 0:
        raise MemoryError("C checker could not allocate its per-head state")
    return o, sT
