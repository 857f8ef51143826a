"""CPU tests of the checker itself: independent derivations, C vs Python, golden fixtures."""
import importlib.util
import os

import numpy as np
import pytest
import torch

from avelang_b200 import synth

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _load_make_golden():
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(GOLDEN, "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("shape,kw", [
    ((1, 256, 4, 4, 64, 64), dict(dtype=torch.float32)),
    ((2, 150, 2, 4, 32, 48), dict(n_states=2, gate_scale=0.01)),
    ((1, 65, 1, 2, 16, 16), dict(n_states=1, gate_scale=0.3)),
    ((1, 1, 1, 1, 8, 8), dict()),
])
def test_three_derivations_agree_fp64(checker, shape, kw):
    O, _ = checker
    i = synth.make_inputs(*shape, seed=11, **kw)
    o1, s1 = O.naive_recurrent_gated_delta_rule(i.q, i.k, i.v, i.g, i.beta, i.scale, i.initial_state)
    o2, s2 = O.chunk_gated_delta_rule_ref(i.q, i.k, i.v, i.g, i.beta, i.scale, i.initial_state)
    o3, s3 = O.affine_gated_delta_rule_ref(i.q, i.k, i.v, i.g, i.beta, i.scale, i.initial_state)
    for o, s in ((o2, s2), (o3, s3)):
        assert O.rel_l2(o, o1) < 1e-12
        assert O.rel_l2(s, s1) < 1e-12


def test_varlen_equals_separate_sequences(checker):
    O, _ = checker
    i = synth.make_inputs(1, 150, 2, 4, 16, 16, seed=5, n_states=3, gate_scale=0.2)
    cu = torch.tensor([0, 1, 70, 150], dtype=torch.int32)
    o, s = O.naive_recurrent_gated_delta_rule(i.q, i.k, i.v, i.g, i.beta, i.scale, i.initial_state, cu)
    oc, sc = O.chunk_gated_delta_rule_ref(i.q, i.k, i.v, i.g, i.beta, i.scale, i.initial_state, cu)
    assert O.rel_l2(oc, o) < 1e-12 and O.rel_l2(sc, s) < 1e-12
    for n in range(3):
        a, b = int(cu[n]), int(cu[n + 1])
        o1, s1 = O.naive_recurrent_gated_delta_rule(i.q[:, a:b], i.k[:, a:b], i.v[:, a:b], i.g[:, a:b], i.beta[:, a:b],
                                                    i.scale, i.initial_state[n:n + 1])
        assert torch.equal(o1[0], o[0, a:b]) and torch.equal(s1[0], s[n])


def test_state_handoff_composes(checker):
    O, _ = checker
    i = synth.make_inputs(1, 100, 2, 2, 16, 16, seed=2, gate_scale=0.1)
    o, s = O.naive_recurrent_gated_delta_rule(i.q, i.k, i.v, i.g, i.beta, i.scale)
    oa, sa = O.naive_recurrent_gated_delta_rule(i.q[:, :37], i.k[:, :37], i.v[:, :37], i.g[:, :37], i.beta[:, :37], i.scale)
    ob, sb = O.naive_recurrent_gated_delta_rule(i.q[:, 37:], i.k[:, 37:], i.v[:, 37:], i.g[:, 37:], i.beta[:, 37:], i.scale, sa)
    assert O.rel_l2(torch.cat([oa, ob], 1), o) < 1e-14 and O.rel_l2(sb, s) < 1e-14


@pytest.mark.parametrize("precision,tol", [("f64", 2e-7), ("f32", 5e-6)])
def test_c_checker_matches_python(checker, precision, tol):
    O, C = checker
    i = synth.make_inputs(1, 190, 2, 4, 64, 64, seed=3, n_states=3, gate_scale=0.3)
    cu = torch.tensor([0, 64, 65, 190], dtype=torch.int32)
    o1, s1 = O.naive_recurrent_gated_delta_rule(i.q, i.k, i.v, i.g, i.beta, i.scale, i.initial_state, cu)
    o2, s2 = C.recurrent(i.q, i.k, i.v, i.g, i.beta, i.scale, i.initial_state, cu, precision=precision)
    assert O.rel_l2(o2, o1) < tol and O.rel_l2(s2, s1) < tol
    o1, s1 = O.naive_recurrent_gated_delta_rule(i.q, i.k, i.v, i.g, i.beta, i.scale, i.initial_state, cu, use_qk_l2norm_in_kernel=True)
    o2, s2 = C.recurrent(i.q, i.k, i.v, i.g, i.beta, i.scale, i.initial_state, cu, precision=precision, use_qk_l2norm_in_kernel=True)
    assert O.rel_l2(o2, o1) < tol and O.rel_l2(s2, s1) < tol


def test_golden_config0(checker):
    O, C = checker
    mg = _load_make_golden()
    gold = np.load(os.path.join(GOLDEN, "config0_fp64.npz"))
    c0 = synth.config0()
    shas = [mg.sha(t) for t in (c0.q, c0.k, c0.v, c0.g, c0.beta)]
    assert shas == list(gold["input_sha"]), "seeded inputs drifted from the fixture"
    o, s = O.naive_recurrent_gated_delta_rule(c0.q, c0.k, c0.v, c0.g, c0.beta, c0.scale)
    assert O.rel_l2(o, torch.from_numpy(gold["o"])) < 1e-6
    assert O.rel_l2(s, torch.from_numpy(gold["final_state"])) < 1e-6
    # the fp32 run of the same recurrence (the CPU baseline) stays close to the fp64 fixture
    o32, s32 = O.naive_recurrent_gated_delta_rule(c0.q, c0.k, c0.v, c0.g, c0.beta, c0.scale, dtype=torch.float32)
    assert O.rel_l2(o32, torch.from_numpy(gold["o"])) < 1e-5
    oc, sc = C.recurrent(c0.q, c0.k, c0.v, c0.g, c0.beta, c0.scale)
    assert O.rel_l2(oc, torch.from_numpy(gold["o"])) < 1e-6 and O.rel_l2(sc, torch.from_numpy(gold["final_state"])) < 1e-6


def test_golden_small_varlen(checker):
    O, C = checker
    mg = _load_make_golden()
    gold = np.load(os.path.join(GOLDEN, "small_varlen_fp64.npz"))
    sm = mg.small_case()
    shas = [mg.sha(t) for t in (sm.q, sm.k, sm.v, sm.g, sm.beta, sm.z, sm.initial_state)]
    assert shas == list(gold["input_sha"])
    o, s = C.recurrent(sm.q, sm.k, sm.v, sm.g, sm.beta, sm.scale, sm.initial_state, sm.cu_seqlens)
    assert O.rel_l2(o, torch.from_numpy(gold["o"])) < 1e-6 and O.rel_l2(s, torch.from_numpy(gold["final_state"])) < 1e-6
    assert O.rel_l2(O.gated_rmsnorm(o, sm.z), torch.from_numpy(gold["y"])) < 1e-6


def test_third_party_opinion(checker, record_property):
    """Import-only cross-check against an installed third-party package, when present (not the reference)."""
    O, _ = checker
    import importlib.metadata as md
    try:
        version = md.version("flash-linear-attention")
    except md.PackageNotFoundError:
        version = "not installed"
    print(f"third opinion: flash-linear-attention {version}")
    naive = pytest.importorskip("fla.ops.gated_delta_rule.naive", reason="third-party package not installed")
    i = synth.make_inputs(2, 96, 4, 4, 32, 48, seed=3, n_states=2, gate_scale=0.3)
    o1, s1 = O.naive_recurrent_gated_delta_rule(i.q, i.k, i.v, i.g, i.beta, i.scale, i.initial_state)
    try:
        o2, s2 = naive.naive_recurrent_gated_delta_rule(i.q.double(), i.k.double(), i.v.double(), i.beta.double(), i.g.double(),
                                                        scale=i.scale, initial_state=i.initial_state.double(), output_final_state=True)
    except Exception as e:  # signature or layout differs in another version: not our contract
        print(f"third opinion: call failed in flash-linear-attention {version}: {e!r} -> no opinion given")
        pytest.skip(f"third-party call failed in flash-linear-attention {version}: {e!r}")
    e_o, e_s = O.rel_l2(o2, o1), O.rel_l2(s2, s1)
    print(f"third opinion: flash-linear-attention {version} answered; o rel-L2 {e_o:.2e}, state rel-L2 {e_s:.2e}")
    record_property("third_opinion", f"flash-linear-attention {version}: o {e_o:.2e}, S {e_s:.2e}")
    assert e_o < 1e-5 and e_s < 1e-5


def test_gated_rmsnorm_properties(checker):
    O, _ = checker
    g = torch.Generator().manual_seed(0)
    x, z = torch.randn(5, 3, 128, generator=g), torch.randn(5, 3, 128, generator=g)
    y = O.gated_rmsnorm(x, z)
    # scale invariance of the normalised part (up to eps) and the gate's sign
    y2 = O.gated_rmsnorm(7.0 * x, z)
    assert O.rel_l2(y2, y) < 1e-5
    ref = x.double() / x.double().pow(2).mean(-1, keepdim=True).add(1e-6).sqrt() * torch.nn.functional.silu(z.double())
    assert O.rel_l2(y, ref) < 1e-14


def test_conv1d_matches_torch_conv(checker):
    O, _ = checker
    g = torch.Generator().manual_seed(0)
    x, w = torch.randn(2, 37, 16, generator=g), torch.randn(16, 4, generator=g)
    y = O.causal_conv1d_silu(x, w)
    ref = torch.nn.functional.conv1d(torch.nn.functional.pad(x.double().transpose(1, 2), (3, 0)), w.double()[:, None, :], groups=16)
    ref = torch.nn.functional.silu(ref).transpose(1, 2)
    assert O.rel_l2(y, ref) < 1e-14
    cu = torch.tensor([0, 2, 20, 37], dtype=torch.int32)
    yv = O.causal_conv1d_silu(x[:1], w, cu)
    for a, b in ((0, 2), (2, 20), (20, 37)):
        assert O.rel_l2(yv[0, a:b], O.causal_conv1d_silu(x[:1, a:b], w)[0]) < 1e-14


def test_varlen_lengths_recipe():
    lens = synth.varlen_lengths()
    assert len(lens) == 64 and sum(lens) == 262144 and min(lens) >= 128 and max(lens) <= 16384
    assert lens == synth.varlen_lengths()
