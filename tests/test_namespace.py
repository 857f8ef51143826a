"""The reference's import spelling and the PyTorch-operator face of the library (no GPU needed for the first two)."""
import pytest
import torch


def test_import_through_the_reference_namespace(built_lib):
    # as in the reference's benchmark/gemm/bench_amdgpu_gemm.py:4 and test/examples/gemm/amdgpu/test_amdgpu_gemm.py:7
    from avelang_kernels import gdn, gemm
    import avelang_kernels.gdn as gdn2
    import avelang_b200.gdn as impl
    assert gdn is gdn2 is impl
    for name in ("chunk_gated_delta_rule", "fused_recurrent_gated_delta_rule", "gated_rmsnorm", "causal_conv1d_silu",
                 "causal_conv1d_update", "gate_beta", "mixed_prefill_decode_step", "read_status"):
        assert callable(getattr(gdn, name)), name
    assert callable(gemm.gemm_pipeline_transposed_b)


def test_operators_are_registered(built_lib):
    from avelang_b200 import torch_ops
    import avelang_kernels  # noqa: F401  (registers the implementations)
    for name in torch_ops.SCHEMAS:
        op = getattr(torch.ops.avelang_gdn, name)
        assert torch._C._dispatch_has_kernel_for_dispatch_key(f"avelang_gdn::{name}", "CUDA"), name
        assert op is not None
    # no CPU kernel is registered: the operators are the CUDA library or nothing
    x = torch.zeros(4, 2, 128, dtype=torch.bfloat16)
    with pytest.raises((NotImplementedError, RuntimeError)):
        torch.ops.avelang_gdn.gated_rmsnorm(x, x, None, 1e-6, False, torch.empty_like(x))


@pytest.mark.gpu
def test_operator_call_matches_public_function(built_lib, checker):
    from avelang_kernels import gdn
    from avelang_b200 import synth
    O, C = checker
    inp = synth.make_inputs(1, 130, 2, 4, 128, 128, seed=2, with_z=True, n_states=1, gate_scale=0.1)
    g = inp.to("cuda")
    o_pub, s_pub = gdn.chunk_gated_delta_rule(g.q, g.k, g.v, g.g, g.beta, initial_state=g.initial_state, output_final_state=True, z=g.z)
    o_op, s_op = torch.empty_like(g.v), torch.empty_like(g.initial_state)
    torch.ops.avelang_gdn.chunk_prefill(g.q, g.k, g.v, g.g, g.beta, o_op, inp.scale, g.initial_state, s_op, None, None, g.z, None,
                                        1e-6, False, 0, None)
    assert torch.equal(o_op, o_pub) and torch.equal(s_op, s_pub)
    o_ref, s_ref = C.recurrent(inp.q, inp.k, inp.v, inp.g, inp.beta, inp.scale, inp.initial_state)
    assert O.rel_l2(o_op.float().cpu(), O.gated_rmsnorm(o_ref, inp.z).to(torch.bfloat16).float()) <= 1e-3
    assert O.rel_l2(s_op.cpu(), s_ref) <= 1e-4
