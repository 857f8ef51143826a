"""CPU tests of the C-ABI boundary: the library loads, exports every declared symbol, the ctypes mirrors
match the C structs, and malformed calls come back as status codes (none of these reaches a kernel)."""
import ctypes
import os
import re
import subprocess

import pytest
import torch

from avelang_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "ave_gdn.h")


def _declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ave_[a-z0-9_]+)\s*\(", text)))


def test_exports_every_declared_symbol(built_lib):
    lib = ctypes.CDLL(built_lib)
    names = _declared_symbols()
    assert len(names) >= 10
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in ave_gdn.h but not exported"
    assert set(names) == set(_lib.SYMBOLS), "ctypes binding and header disagree on the symbol list"


def test_struct_mirrors_match_header(tmp_path):
    src = tmp_path / "sz.c"
    src.write_text('#include "ave_gdn.h"\n#include <stdio.h>\n#include <stddef.h>\nint main(void){printf("%zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu %zu\\n",'
                   "sizeof(AveGdnArgs),sizeof(AveGdnNormArgs),sizeof(AveGemmArgs),sizeof(AveConvArgs),sizeof(AveGateArgs),"
                   "offsetof(AveGdnArgs,scale),offsetof(AveGdnArgs,q_stride_b),sizeof(AveConvUpdateArgs),sizeof(AveGdnDecodeLayerArgs),"
                   "offsetof(AveGdnDecodeLayerArgs,proj_stride),offsetof(AveGemmArgs,status),sizeof(AveGemmReduceArgs),"
                   "offsetof(AveGemmReduceArgs,rows_per_owner));return 0;}\n")
    exe = tmp_path / "sz"
    subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], check=True)
    got = [int(x) for x in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()]
    want = [ctypes.sizeof(_lib.GdnArgs), ctypes.sizeof(_lib.NormArgs), ctypes.sizeof(_lib.GemmArgs),
            ctypes.sizeof(_lib.ConvArgs), ctypes.sizeof(_lib.GateArgs), _lib.GdnArgs.scale.offset,
            _lib.GdnArgs.q_stride_b.offset, ctypes.sizeof(_lib.ConvUpdateArgs), ctypes.sizeof(_lib.DecodeLayerArgs),
            _lib.DecodeLayerArgs.proj_stride.offset, _lib.GemmArgs.status.offset, ctypes.sizeof(_lib.GemmReduceArgs),
            _lib.GemmReduceArgs.rows_per_owner.offset]
    assert got == want


def test_status_codes_without_a_device(built_lib):
    lib = _lib.load()
    assert lib.ave_gdn_abi_version() == _lib.ABI_VERSION == 4
    assert lib.ave_gdn_status_string(0) == b"ok"
    a = _lib.GdnArgs()
    assert lib.ave_gdn_decode_step(ctypes.byref(a), None) == _lib.INVALID_ARGUMENT  # struct_size == 0
    assert lib.ave_gdn_chunk_prefill(None, None) == _lib.INVALID_ARGUMENT
    a.struct_size = ctypes.sizeof(_lib.GdnArgs)
    a.B, a.T, a.Hk, a.Hv, a.dk, a.dv, a.n_seqs, a.chunk = 1, 8, 2, 3, 128, 128, 1, 64
    assert lib.ave_gdn_chunk_prefill(ctypes.byref(a), None) == _lib.INVALID_ARGUMENT  # Hv % Hk
    a.Hv, a.dk = 4, 96
    assert lib.ave_gdn_chunk_prefill(ctypes.byref(a), None) == _lib.UNSUPPORTED
    a.dk = 128
    assert lib.ave_gdn_chunk_prefill(ctypes.byref(a), None) == _lib.INVALID_ARGUMENT  # null tensors
    for n in ("q", "k", "v", "g", "beta", "o"):
        setattr(a, n, 0x1000)
    a.q = 0x1008
    for t in ("q", "k", "v", "o"):
        setattr(a, f"{t}_stride_t", 512); setattr(a, f"{t}_stride_h", 128)
    assert lib.ave_gdn_chunk_prefill(ctypes.byref(a), None) == _lib.MISALIGNED
    a.q = 0x1000
    a.chunk = 32
    assert lib.ave_gdn_chunk_prefill(ctypes.byref(a), None) == _lib.UNSUPPORTED
    a.chunk = 64
    assert lib.ave_gdn_chunk_prefill(ctypes.byref(a), None) == _lib.INVALID_ARGUMENT  # no workspace
    a.workspace, a.workspace_bytes = 0x2000, 16
    assert lib.ave_gdn_chunk_prefill(ctypes.byref(a), None) == _lib.WORKSPACE_TOO_SMALL
    assert lib.ave_gdn_prefill_workspace_bytes(ctypes.byref(a)) > 0
    a.T = 0  # empty input is a no-op, not an error
    assert lib.ave_gdn_chunk_prefill(ctypes.byref(a), None) == _lib.OK
    assert lib.ave_gdn_decode_step(ctypes.byref(a), None) == _lib.OK
    n = _lib.NormArgs()
    n.struct_size = ctypes.sizeof(_lib.NormArgs)
    n.rows, n.d, n.heads = 4, 96, 1
    assert lib.ave_gdn_gated_rmsnorm(ctypes.byref(n), None) == _lib.UNSUPPORTED
    c = _lib.ConvArgs()
    c.struct_size = ctypes.sizeof(_lib.ConvArgs)
    c.B, c.T, c.C, c.width = 1, 4, 16, 5
    assert lib.ave_gdn_conv1d_silu(ctypes.byref(c), None) == _lib.UNSUPPORTED
    g = _lib.GemmArgs()
    g.struct_size = ctypes.sizeof(_lib.GemmArgs)
    g.M, g.N, g.K = 128, 128, 64
    assert lib.ave_gemm_bf16_nt(ctypes.byref(g), None) == _lib.INVALID_ARGUMENT
    r = _lib.GemmReduceArgs()
    r.struct_size = ctypes.sizeof(_lib.GemmReduceArgs)
    r.M, r.N, r.K, r.n_ranks, r.rank, r.rows_per_owner = 256, 128, 64, 2, 0, 64  # two owners of 64 rows cannot hold 256
    assert lib.ave_gemm_bf16_nt_scatter(ctypes.byref(r), None) == _lib.INVALID_ARGUMENT
    assert lib.ave_gemm_reduce_push(ctypes.byref(r), None) == _lib.INVALID_ARGUMENT


def test_status_maps_to_reference_exceptions(built_lib):
    with pytest.raises(ValueError):
        _lib.check(_lib.UNSUPPORTED, "x")
    with pytest.raises(RuntimeError):
        _lib.check(_lib.CUDA_ERROR, "x")
    _lib.check(_lib.OK, "x")


def test_entry_points_validate_like_the_reference(built_lib):
    """Same error behaviour as gemm_pipeline_transposed_b: ValueError naming the offending argument."""
    from avelang_b200 import gdn
    q = torch.zeros(1, 8, 2, 128, dtype=torch.float32)
    with pytest.raises(ValueError, match="q must have dtype torch.bfloat16"):
        gdn.chunk_gated_delta_rule(q, q, q, q, q)
    qb = q.bfloat16()
    with pytest.raises(ValueError, match="CUDA tensor"):
        gdn.chunk_gated_delta_rule(qb, qb, qb, q, q)
    with pytest.raises(ValueError, match="x must have dtype"):
        gdn.gated_rmsnorm(q, q)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setenv("AVE_GDN_LIB", str(tmp_path / "nope.so"))
    monkeypatch.setattr(_lib, "_LIB", None)
    with pytest.raises(ImportError, match="no fallback"):
        _lib.load()
