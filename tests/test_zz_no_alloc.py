"""The no-allocation prefill entry point (scratch in a fixed array inside the library), called through the C ABI
and compared with the regular entry point on two calls in a row.  Kept in a file that sorts last so that a run
stopping at the first failure has already been through every other test."""
import ctypes

import pytest
import torch

from avelang_b200 import _lib, synth

pytestmark = pytest.mark.gpu


def _args(g, o, final, cu):
    a = _lib.GdnArgs()
    a.struct_size = ctypes.sizeof(_lib.GdnArgs)
    a.q, a.k, a.v, a.g, a.beta, a.z, a.o = (t.data_ptr() for t in (g.q, g.k, g.v, g.g, g.beta, g.z, o))
    a.initial_state, a.final_state, a.cu_seqlens = g.initial_state.data_ptr(), final.data_ptr(), cu.data_ptr()
    B, T, Hk, dk = g.q.shape
    Hv, dv = g.v.shape[2:]
    a.B, a.T, a.Hk, a.Hv, a.dk, a.dv, a.n_seqs, a.num_slots, a.chunk = B, T, Hk, Hv, dk, dv, cu.numel() - 1, cu.numel() - 1, 64
    for name, t in (("q", g.q), ("k", g.k), ("v", g.v), ("z", g.z), ("o", o)):
        for d, ax in (("b", 0), ("t", 1), ("h", 2)):
            setattr(a, f"{name}_stride_{d}", t.stride(ax))
    a.g_stride_b, a.g_stride_t = g.g.stride(0), g.g.stride(1)
    a.scale, a.norm_eps = g.scale, 1e-6
    return a


def test_noalloc_prefill_matches_regular_entry_point(built_lib):
    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    for seed, T in ((11, 300), (12, 190)):  # two calls in a row share the one scratch array
        inp = synth.make_inputs(1, T, 2, 4, 128, 128, seed=seed, with_z=True, n_states=3, gate_scale=0.1)
        cu = torch.tensor([0, 70, 71, T], dtype=torch.int32, device="cuda")
        g = inp.to("cuda")
        o_ref, o_new = torch.empty_like(g.v), torch.empty_like(g.v)
        s_ref, s_new = torch.empty_like(g.initial_state), torch.empty_like(g.initial_state)
        a = _args(g, o_ref, s_ref, cu)
        ws = torch.empty(lib.ave_gdn_prefill_workspace_bytes(ctypes.byref(a)), dtype=torch.uint8, device="cuda")
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        assert lib.ave_gdn_chunk_prefill(ctypes.byref(a), stream) == _lib.OK
        b = _args(g, o_new, s_new, cu)  # no workspace given
        assert lib.ave_gdn_chunk_prefill_noalloc(ctypes.byref(b), stream) == _lib.OK
        torch.cuda.synchronize()
        # same kernels on the same inputs: the tolerances of the parity tests (1e-3 / 1e-4) are met with equality
        assert torch.equal(o_new, o_ref) and torch.equal(s_new, s_ref)


def test_noalloc_prefill_long_sequence_against_checker(built_lib, checker):
    """One sequence of 2048 tokens x 4 heads with a gate tensor (about 13 MB of the fixed array): the regular entry point
    cuts such a batch into overlapped launches and parallel parts, the fixed-scratch one runs it as one plain chain on
    the caller's stream, so the two agree within the parity tolerances rather than bit for bit, and both agree with the
    fp64 checker."""
    O, C = checker
    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    inp = synth.make_inputs(1, 2048, 2, 4, 128, 128, seed=13, with_z=True, n_states=1, gate_scale=0.05)
    cu = torch.tensor([0, 2048], dtype=torch.int32, device="cuda")
    g = inp.to("cuda")
    o_ref, o_new = torch.empty_like(g.v), torch.empty_like(g.v)
    s_ref, s_new = torch.empty_like(g.initial_state), torch.empty_like(g.initial_state)
    a = _args(g, o_ref, s_ref, cu)
    ws = torch.empty(lib.ave_gdn_prefill_workspace_bytes(ctypes.byref(a)), dtype=torch.uint8, device="cuda")
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    assert lib.ave_gdn_chunk_prefill(ctypes.byref(a), stream) == _lib.OK
    for _ in range(2):
        b = _args(g, o_new, s_new, cu)
        assert lib.ave_gdn_chunk_prefill_noalloc(ctypes.byref(b), stream) == _lib.OK
    torch.cuda.synchronize()
    o_chk, s_chk = C.recurrent(inp.q, inp.k, inp.v, inp.g, inp.beta, inp.scale, inp.initial_state)
    y_chk = O.gated_rmsnorm(o_chk, inp.z).to(torch.bfloat16).float()
    for o_gpu, s_gpu in ((o_new, s_new), (o_ref, s_ref)):
        assert O.rel_l2(o_gpu.float().cpu(), y_chk) <= 1e-3
        assert O.rel_l2(s_gpu.cpu(), s_chk) <= 1e-4
    assert O.rel_l2(o_new.float().cpu(), o_ref.float().cpu()) <= 1e-3 and O.rel_l2(s_new.cpu(), s_ref.cpu()) <= 1e-4


def test_noalloc_prefill_rejects_oversized_requests(built_lib):
    lib = _lib.load()
    inp = synth.make_inputs(1, 64, 1, 1, 128, 128, seed=1, with_z=True, n_states=1)
    g = inp.to("cuda")
    cu = torch.tensor([0, 64], dtype=torch.int32, device="cuda")
    a = _args(g, torch.empty_like(g.v), torch.empty_like(g.initial_state), cu)
    a.T = 64 * 2000  # about 2000 chunk-heads of scratch: beyond the fixed array; rejected before any launch
    assert lib.ave_gdn_chunk_prefill_noalloc(ctypes.byref(a), torch.cuda.current_stream().cuda_stream) == _lib.WORKSPACE_TOO_SMALL
    with pytest.raises(ValueError, match="workspace too small"):
        _lib.check(_lib.WORKSPACE_TOO_SMALL, "ave_gdn_chunk_prefill_noalloc")
