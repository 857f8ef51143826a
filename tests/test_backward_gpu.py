"""GPU parity of the backward pass (through the C ABI) against automatic differentiation of the fp64 checker."""
import pytest
import torch

from avelang_b200 import synth
from gpu_util import dev

pytestmark = pytest.mark.gpu
BF16_TOL = 1e-3   # gradients returned in bf16, against the checker's gradient rounded to bf16
F32_TOL = 1e-4    # gradients returned in fp32


@pytest.fixture(scope="module")
def gdn(built_lib):
    from avelang_b200 import gdn
    return gdn


def _check(O, got, ref):
    dq, dk, dv, dg, dbeta, ds0 = got
    rq, rk, rv, rg, rb, rs = ref
    for name, x, r in (("dq", dq, rq), ("dk", dk, rk), ("dv", dv, rv)):
        e = O.rel_l2(x.float().cpu(), r.to(torch.bfloat16).float())
        assert e <= BF16_TOL, f"{name}: rel-L2 {e:.3e}"
    for name, x, r in (("dg", dg, rg), ("dbeta", dbeta, rb)):
        e = O.rel_l2(x.cpu(), r)
        assert e <= F32_TOL, f"{name}: rel-L2 {e:.3e}"
    if rs is not None:
        e = O.rel_l2(ds0.cpu(), rs)
        assert e <= F32_TOL, f"d_initial_state: rel-L2 {e:.3e}"


@pytest.mark.parametrize("gate_scale", [1.0, 0.05])
def test_backward_dense_with_states(gdn, checker, gate_scale):
    O, _ = checker
    inp = synth.make_inputs(2, 150, 2, 4, 128, 128, seed=61, n_states=2, gate_scale=gate_scale)
    gen = torch.Generator().manual_seed(62)
    d_o = torch.randn(inp.v.shape, generator=gen).bfloat16()
    d_final = 0.1 * torch.randn(inp.initial_state.shape, generator=gen)
    g = dev(inp)
    got = gdn.gated_delta_rule_backward(g.q, g.k, g.v, g.g, g.beta, d_o.cuda(), inp.scale, g.initial_state, d_final.cuda())
    assert gdn.read_status() == 0
    ref = O.recurrent_grads(inp.q, inp.k, inp.v, inp.g, inp.beta, d_o, inp.scale, inp.initial_state, d_final)
    _check(O, got, ref)


def test_backward_varlen_without_states(gdn, checker):
    O, _ = checker
    inp = synth.make_inputs(1, 260, 2, 4, 128, 128, seed=63, gate_scale=0.2)
    cu = torch.tensor([0, 1, 65, 66, 260], dtype=torch.int32)
    d_o = torch.randn(inp.v.shape, generator=torch.Generator().manual_seed(64)).bfloat16()
    g = dev(inp)
    got = gdn.gated_delta_rule_backward(g.q, g.k, g.v, g.g, g.beta, d_o.cuda(), cu_seqlens=cu.cuda())
    assert got[5] is None and gdn.read_status() == 0
    ref = O.recurrent_grads(inp.q, inp.k, inp.v, inp.g, inp.beta, d_o, inp.scale, None, None, cu)
    _check(O, got, ref)


def test_autograd_function_trains_through_the_chunked_forward(gdn, checker):
    """Forward through the chunked tensor-core kernel, backward through the reverse sweep, via torch.autograd."""
    O, _ = checker
    inp = synth.make_inputs(1, 130, 2, 4, 128, 128, seed=65, n_states=1, gate_scale=0.3)
    g = dev(inp)
    leaves = [t.clone().requires_grad_(True) for t in (g.q, g.k, g.v, g.g, g.beta)]
    s0 = g.initial_state.clone().requires_grad_(True)
    o, final = gdn.GatedDeltaRuleFunction.apply(*leaves, inp.scale, s0)
    gen = torch.Generator().manual_seed(66)
    w_o = torch.randn(o.shape, generator=gen).bfloat16()
    w_s = 0.1 * torch.randn(final.shape, generator=gen)
    ((o.float() * w_o.cuda().float()).sum() + (final * w_s.cuda()).sum()).backward()
    ref = O.recurrent_grads(inp.q, inp.k, inp.v, inp.g, inp.beta, w_o, inp.scale, inp.initial_state, w_s)
    _check(O, (*[t.grad for t in leaves], s0.grad), ref)
