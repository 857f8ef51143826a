"""ctypes binding of libave_gdn_b200.so (declared in include/ave_gdn.h).

The library is the only implementation: when it is missing or cannot be loaded the import of the
entry points fails with an explicit error; there is no CPU or PyTorch fallback."""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
P, U32, I32, I64, U64, F32 = (ctypes.c_void_p, ctypes.c_uint32, ctypes.c_int32, ctypes.c_int64,
                              ctypes.c_uint64, ctypes.c_float)

OK, INVALID_ARGUMENT, UNSUPPORTED, MISALIGNED, CUDA_ERROR, WORKSPACE_TOO_SMALL = range(6)
DEV_BAD_SLOT, DEV_BAD_SEQLEN, DEV_WAIT_EXPIRED = 1, 2, 4
FLAG_QK_L2NORM, FLAG_GATE_FIRST = 1, 2
NOALLOC_SCRATCH_BYTES = 64 << 20
ABI_VERSION = 4


class GdnArgs(ctypes.Structure):
    _fields_ = ([("struct_size", U32), ("flags", U32)]
                + [(n, P) for n in ("q", "k", "v", "g", "beta", "z", "norm_weight", "o", "initial_state",
                                    "final_state", "cu_seqlens", "state_indices", "status", "workspace")]
                + [("workspace_bytes", U64)]
                + [(n, I32) for n in ("B", "T", "Hk", "Hv", "dk", "dv", "n_seqs", "num_slots", "chunk", "max_seqlen")]
                + [(f"{t}_stride_{d}", I64) for t in ("q", "k", "v", "z", "o") for d in ("b", "t", "h")]
                + [("g_stride_b", I64), ("g_stride_t", I64), ("scale", F32), ("norm_eps", F32),
                   ("o_peers", P), ("n_peers", I32), ("reserved1", I32)])


class NormArgs(ctypes.Structure):
    _fields_ = [("struct_size", U32), ("flags", U32), ("x", P), ("z", P), ("weight", P), ("y", P),
                ("rows", I64), ("d", I32), ("heads", I32),
                ("x_stride_t", I64), ("x_stride_h", I64), ("z_stride_t", I64), ("z_stride_h", I64),
                ("y_stride_t", I64), ("y_stride_h", I64), ("eps", F32), ("reserved0", F32)]


class GemmArgs(ctypes.Structure):
    _fields_ = [("struct_size", U32), ("flags", U32), ("a", P), ("b", P), ("c", P),
                ("M", I64), ("N", I64), ("K", I64), ("lda", I64), ("ldb", I64), ("ldc", I64), ("status", P)]


class GemmReduceArgs(ctypes.Structure):
    _fields_ = [("struct_size", U32), ("flags", U32), ("a", P), ("b", P), ("M", I64), ("N", I64), ("K", I64),
                ("lda", I64), ("ldb", I64), ("stage_peers", P), ("stage", P), ("out_peers", P), ("ldc", I64),
                ("n_ranks", I32), ("rank", I32), ("rows_per_owner", I64), ("status", P)]


class ConvArgs(ctypes.Structure):
    _fields_ = [("struct_size", U32), ("flags", U32), ("x", P), ("w", P), ("bias", P), ("y", P), ("cu_seqlens", P),
                ("B", I32), ("T", I32), ("C", I32), ("width", I32), ("n_seqs", I32), ("reserved0", I32),
                ("x_stride_b", I64), ("x_stride_t", I64), ("y_stride_b", I64), ("y_stride_t", I64)]


class ConvUpdateArgs(ctypes.Structure):
    _fields_ = [("struct_size", U32), ("flags", U32), ("x", P), ("w", P), ("bias", P), ("y", P), ("conv_state", P),
                ("state_indices", P), ("n_seqs", I32), ("C", I32), ("width", I32), ("num_slots", I32),
                ("x_stride", I64), ("y_stride", I64), ("status", P)]


class DecodeLayerArgs(ctypes.Structure):
    _fields_ = ([("struct_size", U32), ("flags", U32)]
                + [(n, P) for n in ("proj", "conv_w", "conv_bias", "conv_state", "A_log", "dt_bias", "norm_weight", "state_pool",
                                    "state_indices", "o", "status")]
                + [(n, I32) for n in ("n_seqs", "Hk", "Hv", "dk", "dv", "width", "num_slots", "reserved0")]
                + [("proj_stride", I64), ("o_stride", I64), ("scale", F32), ("norm_eps", F32)])


class BwdArgs(ctypes.Structure):
    _fields_ = ([("struct_size", U32), ("flags", U32)]
                + [(n, P) for n in ("q", "k", "v", "g", "beta", "d_o", "initial_state", "d_final_state", "cu_seqlens", "d_q", "d_k",
                                    "d_v", "d_g", "d_beta", "d_initial_state", "status", "workspace")]
                + [("workspace_bytes", U64)]
                + [(n, I32) for n in ("B", "T", "Hk", "Hv", "dk", "dv", "n_seqs", "reserved0")]
                + [(f"{t}_stride_{d}", I64) for t in ("q", "k", "v", "do") for d in ("b", "t", "h")]
                + [("g_stride_b", I64), ("g_stride_t", I64), ("scale", F32), ("reserved1", F32)])


class GateArgs(ctypes.Structure):
    _fields_ = [("struct_size", U32), ("flags", U32), ("a", P), ("b", P), ("A_log", P), ("dt_bias", P),
                ("g", P), ("beta", P), ("rows", I64), ("Hv", I32), ("reserved0", I32),
                ("a_stride_row", I64), ("b_stride_row", I64)]


# every symbol include/ave_gdn.h declares: name -> (restype, argtypes)
SYMBOLS = {
    "ave_gdn_chunk_prefill": (ctypes.c_int, [ctypes.POINTER(GdnArgs), P]),
    "ave_gdn_prefill_workspace_bytes": (ctypes.c_size_t, [ctypes.POINTER(GdnArgs)]),
    "ave_gdn_prefill_launch_count": (ctypes.c_int, [ctypes.POINTER(GdnArgs)]),
    "ave_gdn_chunk_prefill_noalloc": (ctypes.c_int, [ctypes.POINTER(GdnArgs), P]),
    "ave_gdn_decode_step": (ctypes.c_int, [ctypes.POINTER(GdnArgs), P]),
    "ave_gdn_gated_rmsnorm": (ctypes.c_int, [ctypes.POINTER(NormArgs), P]),
    "ave_gemm_bf16_nt": (ctypes.c_int, [ctypes.POINTER(GemmArgs), P]),
    "ave_gemm_bf16_nt_scatter": (ctypes.c_int, [ctypes.POINTER(GemmReduceArgs), P]),
    "ave_gemm_reduce_push": (ctypes.c_int, [ctypes.POINTER(GemmReduceArgs), P]),
    "ave_gdn_conv1d_silu": (ctypes.c_int, [ctypes.POINTER(ConvArgs), P]),
    "ave_gdn_conv1d_update": (ctypes.c_int, [ctypes.POINTER(ConvUpdateArgs), P]),
    "ave_gdn_gate_beta": (ctypes.c_int, [ctypes.POINTER(GateArgs), P]),
    "ave_gdn_decode_layer_step": (ctypes.c_int, [ctypes.POINTER(DecodeLayerArgs), P]),
    "ave_gdn_recurrent_backward": (ctypes.c_int, [ctypes.POINTER(BwdArgs), P]),
    "ave_gdn_backward_workspace_bytes": (ctypes.c_size_t, [ctypes.POINTER(BwdArgs)]),
    "ave_gdn_abi_version": (ctypes.c_int, []),
    "ave_gdn_status_string": (ctypes.c_char_p, [ctypes.c_int]),
    "ave_gdn_last_cuda_error": (ctypes.c_int, []),
}

_LIB = None


def lib_path() -> str:
    return os.environ.get("AVE_GDN_LIB", os.path.join(_HERE, "libave_gdn_b200.so"))


def load():
    """Load the shared library once; raises if it is absent (build it with `python -m avelang_b200.build`)."""
    global _LIB
    if _LIB is None:
        path = lib_path()
        if not os.path.exists(path):
            raise ImportError(f"{path} is missing: run `python -m avelang_b200.build` (needs nvcc); "
                              "this package has no fallback implementation")
        lib = ctypes.CDLL(path)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        if lib.ave_gdn_abi_version() != ABI_VERSION:
            raise ImportError("libave_gdn_b200.so has an unexpected ABI version")
        _LIB = lib
    return _LIB


def check(rc: int, what: str) -> None:
    """Map a status code to the reference's exception convention: argument problems raise ValueError
    (python/avelang_kernels/amdgpu_gemm.py:463-486), device/runtime problems RuntimeError
    (python/avelang/backends/nvidia/driver.py:68-83)."""
    if rc == OK:
        return
    lib = load()
    msg = f"{what}: {lib.ave_gdn_status_string(rc).decode()}"
    if rc in (INVALID_ARGUMENT, UNSUPPORTED, MISALIGNED, WORKSPACE_TOO_SMALL):
        raise ValueError(msg)
    raise RuntimeError(f"{msg} (cudaError {lib.ave_gdn_last_cuda_error()})")
