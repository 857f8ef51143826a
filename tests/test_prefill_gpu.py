"""GPU parity of the chunked prefill (through the C ABI) against the CPU checker."""
import numpy as np
import os
import pytest
import torch

from avelang_b200 import synth
from gpu_util import check_o, check_s, dev

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def gdn(built_lib):
    from avelang_b200 import gdn
    return gdn


def _run(gdn, inp, **kw):
    g = dev(inp)
    o, s = gdn.chunk_gated_delta_rule(g.q, g.k, g.v, g.g, g.beta, initial_state=g.initial_state,
                                      output_final_state=True,
                                      cu_seqlens=g.cu_seqlens if inp.cu_seqlens is not None else None, **kw)
    return o, s


@pytest.mark.parametrize("T", [1, 63, 64, 65, 127, 128, 129, 200])
@pytest.mark.parametrize("gate_scale", [1.0, 0.01])
def test_prefill_lengths(gdn, checker, T, gate_scale):
    O, C = checker
    inp = synth.make_inputs(2, T, 2, 4, 128, 128, seed=T, n_states=2, gate_scale=gate_scale)
    o, s = _run(gdn, inp)
    o_ref, s_ref = C.recurrent(inp.q, inp.k, inp.v, inp.g, inp.beta, inp.scale, inp.initial_state)
    check_o(O, o, o_ref)
    check_s(O, s, s_ref)


def test_prefill_config0_shape_against_golden(gdn, checker):
    """B=1, T=256, 4 heads, d=64.  The fixture is the fp64 run on the fp32 inputs; the kernel consumes the
    same inputs rounded to bf16, so it is compared with the checker on the rounded inputs, and the fixture
    pins the checker."""
    O, C = checker
    c0 = synth.config0()
    gold = np.load(os.path.join(GOLDEN, "config0_fp64.npz"))
    o64, s64 = C.recurrent(c0.q, c0.k, c0.v, c0.g, c0.beta, c0.scale)
    assert O.rel_l2(o64, torch.from_numpy(gold["o"])) < 1e-6
    inp = synth.make_inputs(1, 256, 4, 4, 64, 64, seed=0)  # same draws, rounded to bf16
    o, s = _run(gdn, inp)
    o_ref, s_ref = C.recurrent(inp.q, inp.k, inp.v, inp.g, inp.beta, inp.scale)
    check_o(O, o, o_ref)
    check_s(O, s, s_ref)
    # rounding q/k/v to bf16 moves the result by ~bf16 epsilon, not more
    assert O.rel_l2(o.float().cpu(), torch.from_numpy(gold["o"])) < 2e-2


def test_prefill_golden_small_varlen_fused_norm(gdn, checker):
    O, _ = checker
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(GOLDEN, "make_golden.py"))
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    sm = mg.small_case()
    gold = np.load(os.path.join(GOLDEN, "small_varlen_fp64.npz"))
    g = dev(sm)
    o, s = gdn.chunk_gated_delta_rule(g.q, g.k, g.v, g.g, g.beta, initial_state=g.initial_state,
                                      output_final_state=True, cu_seqlens=g.cu_seqlens)
    check_o(O, o, torch.from_numpy(gold["o"]))
    check_s(O, s, torch.from_numpy(gold["final_state"]))
    y, _ = gdn.chunk_gated_delta_rule(g.q, g.k, g.v, g.g, g.beta, initial_state=g.initial_state,
                                      cu_seqlens=g.cu_seqlens, z=g.z)
    check_o(O, y, torch.from_numpy(gold["y"]))


def test_prefill_varlen_ragged_l2norm_strided_heads(gdn, checker):
    """Packed ragged sequences, in-kernel q/k normalisation, and a head-sharded (strided) view of the
    packed tensors: the shard's result must equal the same heads of the unsharded run."""
    O, C = checker
    inp = synth.make_inputs(1, 700, 4, 8, 128, 128, seed=21, n_states=6, gate_scale=0.05, l2norm=False)
    cu = torch.tensor([0, 1, 64, 129, 130, 450, 700], dtype=torch.int32)
    inp.cu_seqlens = cu
    o, s = _run(gdn, inp, use_qk_l2norm_in_kernel=True)
    o_ref, s_ref = C.recurrent(inp.q, inp.k, inp.v, inp.g, inp.beta, inp.scale, inp.initial_state, cu,
                               use_qk_l2norm_in_kernel=True)
    check_o(O, o, o_ref)
    check_s(O, s, s_ref)
    g = dev(inp)
    ks, vs = slice(2, 4), slice(4, 8)  # second half of the heads, as one rank of two would own them
    o2, s2 = gdn.chunk_gated_delta_rule(g.q[:, :, ks], g.k[:, :, ks], g.v[:, :, vs], g.g[:, :, vs].contiguous(),
                                        g.beta[:, :, vs].contiguous(), initial_state=g.initial_state[:, vs].contiguous(),
                                        output_final_state=True, use_qk_l2norm_in_kernel=True, cu_seqlens=g.cu_seqlens)
    assert torch.equal(o2, o[:, :, vs]) and torch.equal(s2, s[:, vs])


def test_prefill_state_handoff_and_decode_agreement(gdn, checker):
    """prefill(T) == prefill(T1) -> state -> prefill(T2), and the chunked kernel agrees with the
    token-by-token kernel on the same inputs."""
    O, C = checker
    inp = synth.make_inputs(2, 300, 2, 4, 128, 128, seed=33, n_states=2, gate_scale=0.02)
    g = dev(inp)
    o, s = gdn.chunk_gated_delta_rule(g.q, g.k, g.v, g.g, g.beta, initial_state=g.initial_state, output_final_state=True)
    cut = 128
    oa, sa = gdn.chunk_gated_delta_rule(g.q[:, :cut], g.k[:, :cut], g.v[:, :cut], g.g[:, :cut], g.beta[:, :cut],
                                        initial_state=g.initial_state, output_final_state=True)
    ob, sb = gdn.chunk_gated_delta_rule(g.q[:, cut:], g.k[:, cut:], g.v[:, cut:], g.g[:, cut:], g.beta[:, cut:],
                                        initial_state=sa, output_final_state=True)
    assert O.rel_l2(torch.cat([oa, ob], 1).float().cpu(), o.float().cpu()) < 1e-3
    assert O.rel_l2(sb.cpu(), s.cpu()) < 1e-5
    orr, sr = gdn.fused_recurrent_gated_delta_rule(g.q, g.k, g.v, g.g, g.beta, initial_state=g.initial_state)
    assert O.rel_l2(o.float().cpu(), orr.float().cpu()) < 2e-3
    assert O.rel_l2(s.cpu(), sr.cpu()) < 1e-4


def test_prefill_state_indices_pool_in_place(gdn, checker):
    O, C = checker
    inp = synth.make_inputs(1, 260, 2, 4, 128, 128, seed=5, n_states=3, gate_scale=0.05)
    cu = torch.tensor([0, 100, 101, 260], dtype=torch.int32)
    g = dev(inp)
    pool = torch.randn(6, 4, 128, 128, device="cuda") * 0.02
    idx = torch.tensor([4, -1, 1], dtype=torch.int32, device="cuda")
    pool0 = pool.clone()
    o, st = gdn.chunk_gated_delta_rule(g.q, g.k, g.v, g.g, g.beta, initial_state=pool, output_final_state=True,
                                       cu_seqlens=cu.cuda(), state_indices=idx)
    assert st.data_ptr() == pool.data_ptr() and gdn.read_status() == 0
    for n, slot in ((0, 4), (2, 1)):
        a, b = int(cu[n]), int(cu[n + 1])
        o_ref, s_ref = C.recurrent(inp.q[:, a:b], inp.k[:, a:b], inp.v[:, a:b], inp.g[:, a:b], inp.beta[:, a:b], inp.scale,
                                   pool0[slot:slot + 1].cpu())
        check_o(O, o[:, a:b], o_ref)
        check_s(O, pool[slot:slot + 1], s_ref)
    assert torch.count_nonzero(o[:, 100:101]) == 0
    for slot in (0, 2, 3, 5):
        assert torch.equal(pool[slot], pool0[slot])


def test_prefill_empty_and_deterministic(gdn):
    z = torch.zeros(1, 0, 2, 128, dtype=torch.bfloat16, device="cuda")
    zg = torch.zeros(1, 0, 2, dtype=torch.float32, device="cuda")
    o, s = gdn.chunk_gated_delta_rule(z, z, z, zg, zg)
    assert o.shape == (1, 0, 2, 128) and s is None
    inp = synth.make_inputs(1, 333, 2, 4, 128, 128, seed=8, n_states=1)
    a = _run(gdn, inp)
    b = _run(gdn, inp)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]), "two runs differ: a race"


def test_prefill_config1_full_size(gdn, checker):
    """B=1, T=8192, 16 key / 32 value heads, d=128, fused gated RMSNorm, against the C checker (fp64)."""
    O, C = checker
    inp = synth.config1()
    g = dev(inp)
    y, s = gdn.chunk_gated_delta_rule(g.q, g.k, g.v, g.g, g.beta, output_final_state=True, z=g.z)
    o_ref, s_ref = C.recurrent(inp.q, inp.k, inp.v, inp.g, inp.beta, inp.scale)
    check_o(O, y, O.gated_rmsnorm(o_ref, inp.z))
    check_s(O, s, s_ref)
    inp = synth.config1(T=2048, gate_scale=0.01)  # slow gate: the inter-chunk state path dominates
    g = dev(inp)
    y, s = gdn.chunk_gated_delta_rule(g.q, g.k, g.v, g.g, g.beta, output_final_state=True, z=g.z)
    o_ref, s_ref = C.recurrent(inp.q, inp.k, inp.v, inp.g, inp.beta, inp.scale)
    check_o(O, y, O.gated_rmsnorm(o_ref, inp.z))
    check_s(O, s, s_ref)


def test_prefill_config3_varlen_sample(gdn, checker):
    """Packed varlen batch with the recipe of the 256K-token configuration at 1/8 of the tokens
    (64 sequences, log-uniform lengths, nonzero initial states): a sample of sequences against the checker."""
    O, C = checker
    inp = synth.config3(total=32768, lo=128, hi=2048)
    o, s = _run(gdn, inp)
    cu = inp.cu_seqlens.tolist()
    lens = inp.extras["lengths"]
    order = sorted(range(64), key=lambda n: lens[n])
    for n in (order[0], order[31], order[-1]):
        a, b = cu[n], cu[n + 1]
        o_ref, s_ref = C.recurrent(inp.q[:, a:b], inp.k[:, a:b], inp.v[:, a:b], inp.g[:, a:b], inp.beta[:, a:b], inp.scale,
                                   inp.initial_state[n:n + 1])
        check_o(O, o[:, a:b], o_ref)
        check_s(O, s[n:n + 1], s_ref)


def test_prefill_config3_full_size(gdn, checker):
    """The 256K-token packed varlen configuration at full size (64 sequences of 128..16384 tokens, nonzero initial
    states): every sequence and every final state against the C checker, and a second run bit-identical (the scan
    walks the sequences longest first; the order must not leak into results)."""
    O, C = checker
    inp = synth.config3()
    o, s = _run(gdn, inp)
    o2, s2 = _run(gdn, inp)
    assert torch.equal(o, o2) and torch.equal(s, s2)
    cu = inp.cu_seqlens.tolist()
    lens = inp.extras["lengths"]
    assert sum(lens) == inp.q.shape[1] == cu[-1]
    o_ref, s_ref = C.recurrent(inp.q, inp.k, inp.v, inp.g, inp.beta, inp.scale, inp.initial_state, inp.cu_seqlens)
    o_cpu, s_cpu = o.cpu(), s.cpu()
    for n in range(64):
        a, b = cu[n], cu[n + 1]
        check_o(O, o_cpu[:, a:b], o_ref[:, a:b])
        check_s(O, s_cpu[n:n + 1], s_ref[n:n + 1])
    check_o(O, o_cpu, o_ref)
    check_s(O, s_cpu, s_ref)


@pytest.mark.parametrize("gate_scale", [1.0, 0.01, 0.001])
@pytest.mark.parametrize("with_z", [False, True])
def test_prefill_parallel_parts_dense(gdn, checker, gate_scale, with_z):
    """Few long chains (2 sequences x 4 heads, 65 chunks with a ragged tail): each sequence is cut into parts that are
    scanned at the same time (a local and a transition chain per later part), combined, and fixed up by one GEMM per
    part.  Slow gates make the state that crosses the parts the dominant term."""
    O, C = checker
    T = 64 * 64 + 37
    inp = synth.make_inputs(2, T, 2, 4, 128, 128, seed=41, with_z=with_z, n_states=2, gate_scale=gate_scale)
    g = dev(inp)
    o, s = gdn.chunk_gated_delta_rule(g.q, g.k, g.v, g.g, g.beta, initial_state=g.initial_state, output_final_state=True,
                                      z=g.z if with_z else None)
    assert gdn.read_status() == 0
    o_ref, s_ref = C.recurrent(inp.q, inp.k, inp.v, inp.g, inp.beta, inp.scale, inp.initial_state)
    if with_z:
        o_ref = O.gated_rmsnorm(o_ref, inp.z)
    for t0 in range(0, T, 1024):  # per stretch of tokens, so that one wrong part cannot hide in the total
        check_o(O, o[:, t0:t0 + 1024], o_ref[:, t0:t0 + 1024])
    check_s(O, s, s_ref)


def test_prefill_parallel_parts_varlen_pool(gdn, checker):
    """Packed sequences of very different lengths with pool slots: long ones are cut into parts, short ones stay plain
    chains, one is skipped by a negative slot; with and without the max_seqlen bound."""
    O, C = checker
    lens = [5000, 64, 1, 2049, 3100]
    T = sum(lens)
    inp = synth.make_inputs(1, T, 2, 4, 128, 128, seed=43, with_z=True, n_states=8, gate_scale=0.01)
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    idx = torch.tensor([6, 1, 3, -1, 0], dtype=torch.int32)
    g = dev(inp)
    for z in (None, g.z):
        for bound in (None, max(lens)):
            pool = g.initial_state.clone()
            o, _ = gdn.chunk_gated_delta_rule(g.q, g.k, g.v, g.g, g.beta, initial_state=pool, output_final_state=True,
                                              cu_seqlens=cu.cuda(), state_indices=idx.cuda(), z=z, max_seqlen=bound)
            assert gdn.read_status() == 0
            for n, L in enumerate(lens):
                a, b = int(cu[n]), int(cu[n + 1])
                sl = int(idx[n])
                if sl < 0:
                    assert torch.count_nonzero(o[:, a:b]) == 0
                    continue
                o_ref, s_ref = C.recurrent(inp.q[:, a:b], inp.k[:, a:b], inp.v[:, a:b], inp.g[:, a:b], inp.beta[:, a:b], inp.scale,
                                           inp.initial_state[sl:sl + 1])
                check_o(O, o[:, a:b], o_ref if z is None else O.gated_rmsnorm(o_ref, inp.z[:, a:b]))
                check_s(O, pool[sl:sl + 1], s_ref)
            unused = [sl for sl in range(8) if sl not in idx.tolist()]
            assert torch.equal(pool[unused].cpu(), inp.initial_state[unused])


def test_prefill_rejects_a_non_monotone_offset_table(gdn):
    """Offsets that are valid pair by pair but not as a whole would need more chunks than the scratch holds: the whole
    batch is skipped and flagged, nothing is read or written out of bounds, and the next call works."""
    inp = synth.make_inputs(1, 8192, 2, 4, 128, 128, seed=3, n_states=3)
    g = dev(inp)
    bad = torch.tensor([0, 5000, 3000, 8192], dtype=torch.int32, device="cuda")
    s_in = g.initial_state.clone()
    gdn.chunk_gated_delta_rule(g.q, g.k, g.v, g.g, g.beta, initial_state=s_in, output_final_state=True, cu_seqlens=bad)
    assert gdn.read_status() & 2  # AVE_GDN_DEV_BAD_SEQLEN
    assert torch.equal(s_in, g.initial_state)
    good = torch.tensor([0, 3000, 5000, 8192], dtype=torch.int32, device="cuda")
    o, s = gdn.chunk_gated_delta_rule(g.q, g.k, g.v, g.g, g.beta, initial_state=s_in, output_final_state=True, cu_seqlens=good)
    assert gdn.read_status() == 0 and bool(torch.isfinite(o.float()).all())


def test_prefill_two_host_threads_two_streams(gdn, checker):
    """Two host threads enqueue range-overlapped prefills on their own streams at the same time (the schedule forks onto
    helper streams through events): both results match the checker."""
    import threading
    O, C = checker
    inps = [synth.make_inputs(1, 4096, 2, 4, 128, 128, seed=50 + i, with_z=True, n_states=1, gate_scale=0.05) for i in range(2)]
    gs = [dev(i) for i in inps]
    res, errs = [None, None], []

    def work(i):
        try:
            st = torch.cuda.Stream()
            with torch.cuda.stream(st):
                for _ in range(4):
                    res[i] = gdn.chunk_gated_delta_rule(gs[i].q, gs[i].k, gs[i].v, gs[i].g, gs[i].beta,
                                                        initial_state=gs[i].initial_state, output_final_state=True, z=gs[i].z)
            st.synchronize()
        except Exception as e:  # surfaced in the main thread
            errs.append(e)

    th = [threading.Thread(target=work, args=(i,)) for i in range(2)]
    [t.start() for t in th]
    [t.join() for t in th]
    assert not errs, errs
    torch.cuda.synchronize()
    assert gdn.read_status() == 0
    for i in range(2):
        o_ref, s_ref = C.recurrent(inps[i].q, inps[i].k, inps[i].v, inps[i].g, inps[i].beta, inps[i].scale, inps[i].initial_state)
        check_o(O, res[i][0], O.gated_rmsnorm(o_ref, inps[i].z))
        check_s(O, res[i][1], s_ref)


def test_mixed_prefill_decode_step(gdn, checker):
    """A continuous-batching step: five single-token (decode) sequences followed by three prefill sequences in one
    packed batch, all states in slots of one pool, fused gated norm.  Every sequence is held against the checker run
    from its slot's state; slots no sequence uses stay untouched."""
    O, C = checker
    lens = [1, 1, 1, 1, 1, 70, 128, 33]
    T, n_dec, n_slots = sum(lens), 5, 12
    inp = synth.make_inputs(1, T, 2, 4, 128, 128, seed=21, with_z=True, n_states=n_slots, gate_scale=0.3)
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    slots = torch.tensor([7, 2, 11, 0, 5, 9, 3, 6], dtype=torch.int32)
    g = dev(inp)
    pool = g.initial_state.clone()
    o = gdn.mixed_prefill_decode_step(g.q, g.k, g.v, g.g, g.beta, cu.cuda(), n_dec, pool, slots.cuda(), z=g.z)
    assert gdn.read_status() == 0
    for n, L in enumerate(lens):
        a, b = int(cu[n]), int(cu[n + 1])
        sl = int(slots[n])
        o_ref, s_ref = C.recurrent(inp.q[:, a:b], inp.k[:, a:b], inp.v[:, a:b], inp.g[:, a:b], inp.beta[:, a:b], inp.scale,
                                   inp.initial_state[sl:sl + 1])
        check_o(O, o[:, a:b], O.gated_rmsnorm(o_ref, inp.z[:, a:b]))
        check_s(O, pool[sl:sl + 1], s_ref)
    unused = [s for s in range(n_slots) if s not in slots.tolist()]
    assert torch.equal(pool[unused].cpu(), inp.initial_state[unused])
    with pytest.raises(ValueError):
        gdn.mixed_prefill_decode_step(g.q, g.k, g.v, g.g, g.beta, cu.cuda(), 99, pool, slots.cuda())


def test_prefill_varlen_max_seqlen_hint(gdn, checker):
    """With the longest sequence known, the chunk ranges of a packed batch of few long chains (16 sequences x 4 heads)
    are sized from it; results are bit-identical to the schedule sized from the packed total, and a sequence longer
    than the stated bound is skipped and flagged."""
    O, C = checker
    inp = synth.config3(n_seqs=16, total=32768, lo=128, hi=8192, Hk=2, Hv=4)
    lens = inp.extras["lengths"]
    o0, s0 = _run(gdn, inp)
    o1, s1 = _run(gdn, inp, max_seqlen=max(lens))
    assert gdn.read_status() == 0
    assert torch.equal(o0, o1) and torch.equal(s0, s1)
    n = max(range(16), key=lambda i: lens[i])
    a, b = int(inp.cu_seqlens[n]), int(inp.cu_seqlens[n + 1])
    o_ref, s_ref = C.recurrent(inp.q[:, a:b], inp.k[:, a:b], inp.v[:, a:b], inp.g[:, a:b], inp.beta[:, a:b], inp.scale,
                               inp.initial_state[n:n + 1])
    check_o(O, o1[:, a:b], o_ref)
    check_s(O, s1[n:n + 1], s_ref)
    _run(gdn, inp, max_seqlen=max(lens) - 1)
    assert gdn.read_status() & 2  # AVE_GDN_DEV_BAD_SEQLEN
