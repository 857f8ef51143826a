"""GPU parity of the fused recurrent step (through the C ABI) against the CPU checker."""
import pytest
import torch

from avelang_b200 import synth
from gpu_util import check_o, check_s, dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gdn(built_lib):
    from avelang_b200 import gdn
    return gdn


@pytest.mark.parametrize("d,Hk,Hv", [(128, 2, 4), (64, 2, 2), (128, 3, 3)])
def test_decode_step_slot_pool(gdn, checker, d, Hk, Hv):
    O, C = checker
    inp = synth.config2(seed=1, n_seqs=24, n_slots=40, Hk=Hk, Hv=Hv, d=d)
    idx = inp.state_indices.clone()
    idx[3] = -1  # skipped sequence
    pool0 = inp.state_pool.clone()
    g = dev(inp)
    pool = g.state_pool.clone()
    o, st = gdn.fused_recurrent_gated_delta_rule(g.q, g.k, g.v, g.g, g.beta, initial_state=pool,
                                                 state_indices=idx.cuda())
    assert st.data_ptr() == pool.data_ptr()
    assert gdn.read_status() == 0
    live = [n for n in range(24) if idx[n] >= 0]
    s0 = pool0[idx[live].long()]
    sel = lambda t: t[live]
    o_ref, s_ref = C.recurrent(sel(inp.q), sel(inp.k), sel(inp.v), sel(inp.g), sel(inp.beta), inp.scale, s0)
    check_o(O, o[live], o_ref)
    check_s(O, pool[idx[live].long()], s_ref)
    assert torch.count_nonzero(o[3]) == 0
    untouched = torch.ones(40, dtype=torch.bool)
    untouched[idx[live].long()] = False
    assert torch.equal(pool.cpu()[untouched], pool0[untouched]), "slots outside state_indices were modified"


def test_decode_chain_of_steps_matches_recurrence(gdn, checker):
    """1000 chained single-token steps on the same slots == one 1000-token recurrence (slow gate, so the
    state really carries over)."""
    O, C = checker
    steps, N, Hk, Hv, d = 1000, 3, 1, 2, 128
    inp = synth.make_inputs(N, steps, Hk, Hv, d, d, seed=4, n_states=N, gate_scale=0.01)
    g = dev(inp)
    pool = torch.zeros(8, Hv, d, d, device="cuda")
    idx = torch.tensor([5, 0, 2], dtype=torch.int32, device="cuda")
    pool[idx.long()] = g.initial_state
    outs = []
    for t in range(steps):
        o, _ = gdn.fused_recurrent_gated_delta_rule(g.q[:, t:t + 1], g.k[:, t:t + 1], g.v[:, t:t + 1], g.g[:, t:t + 1],
                                                    g.beta[:, t:t + 1], initial_state=pool, state_indices=idx)
        outs.append(o)
    o_ref, s_ref = C.recurrent(inp.q, inp.k, inp.v, inp.g, inp.beta, inp.scale, inp.initial_state)
    check_o(O, torch.cat(outs, 1), o_ref)
    check_s(O, pool[idx.long()], s_ref)
    # the multi-token form (state kept in registers across tokens) agrees with the chained single-token steps
    o2, s2 = gdn.fused_recurrent_gated_delta_rule(g.q, g.k, g.v, g.g, g.beta, initial_state=g.initial_state)
    assert O.rel_l2(o2.float().cpu(), torch.cat(outs, 1).float().cpu()) < 1e-3
    assert O.rel_l2(s2.cpu(), pool[idx.long()].cpu()) < 1e-5


def test_decode_varlen_l2norm_and_fused_norm(gdn, checker):
    O, C = checker
    inp = synth.make_inputs(1, 90, 2, 4, 128, 128, seed=9, with_z=True, n_states=3, gate_scale=0.1, l2norm=False)
    cu = torch.tensor([0, 1, 50, 90], dtype=torch.int32)
    g = dev(inp)
    w = torch.linspace(0.5, 1.5, 128)
    o, s = gdn.fused_recurrent_gated_delta_rule(g.q, g.k, g.v, g.g, g.beta, initial_state=g.initial_state,
                                                use_qk_l2norm_in_kernel=True, cu_seqlens=cu.cuda(), z=g.z,
                                                norm_weight=w.cuda())
    o_ref, s_ref = C.recurrent(inp.q, inp.k, inp.v, inp.g, inp.beta, inp.scale, inp.initial_state, cu,
                               use_qk_l2norm_in_kernel=True)
    check_o(O, o, O.gated_rmsnorm(o_ref, inp.z, w))
    check_s(O, s, s_ref)


def test_decode_bad_slot_is_reported_not_faulted(gdn):
    inp = synth.config2(seed=2, n_seqs=4, n_slots=4, Hk=1, Hv=2, d=128)
    g = dev(inp)
    idx = torch.tensor([0, 7, 1, 2], dtype=torch.int32, device="cuda")  # 7 is outside the pool
    pool = g.state_pool.clone()
    o, _ = gdn.fused_recurrent_gated_delta_rule(g.q, g.k, g.v, g.g, g.beta, initial_state=pool, state_indices=idx)
    assert gdn.read_status() & 1
    assert gdn.read_status() == 0
    assert torch.count_nonzero(o[1]) == 0 and torch.equal(pool[3], g.state_pool[3])


def test_decode_full_size_step_properties(gdn, checker):
    """Full 256-sequence, 32-head step over a 512-slot pool: a sample of tiles against the checker, and
    untouched slots stay bit-identical."""
    O, C = checker
    inp = synth.config2()
    g = dev(inp)
    pool = g.state_pool.clone()
    o, _ = gdn.fused_recurrent_gated_delta_rule(g.q, g.k, g.v, g.g, g.beta, initial_state=pool,
                                                state_indices=g.state_indices)
    # every one of the 256 sequences, and each one on its own so that a wrong slot cannot hide in the total
    idx = inp.state_indices.long()
    o_ref, s_ref = C.recurrent(inp.q, inp.k, inp.v, inp.g, inp.beta, inp.scale, inp.state_pool[idx])
    o_cpu, s_cpu = o.float().cpu(), pool[g.state_indices.long()].cpu()
    o_ref16 = o_ref.to(torch.bfloat16).float()
    for n in range(256):
        assert O.rel_l2(o_cpu[n], o_ref16[n]) <= 1e-3 and O.rel_l2(s_cpu[n], s_ref[n]) <= 1e-4, n
    check_o(O, o, o_ref)
    check_s(O, s_cpu, s_ref)
    untouched = torch.ones(512, dtype=torch.bool)
    untouched[inp.state_indices.long()] = False
    assert torch.equal(pool[untouched.cuda()], g.state_pool[untouched.cuda()])


def test_prefill_into_pool_then_decode_matches_recurrence(gdn, checker):
    """Continuous batching hand-off: the chunked prefill writes its final states straight into pool slots, decode
    steps continue from those slots, and the whole thing equals one token recurrence over prompt + generated tokens."""
    O, C = checker
    Tp, Td, N, Hk, Hv, d = 150, 20, 2, 2, 4, 128
    inp = synth.make_inputs(N, Tp + Td, Hk, Hv, d, d, seed=6, gate_scale=0.05)
    g = dev(inp)
    pool = torch.zeros(5, Hv, d, d, device="cuda")
    idx = torch.tensor([3, 1], dtype=torch.int32, device="cuda")
    # prefill the prompts as one packed batch
    pk = lambda t: t[:, :Tp].reshape(1, N * Tp, *t.shape[2:]).contiguous()
    cu = torch.tensor([0, Tp, 2 * Tp], dtype=torch.int32, device="cuda")
    o_p, st = gdn.chunk_gated_delta_rule(pk(g.q), pk(g.k), pk(g.v), pk(g.g), pk(g.beta), initial_state=pool,
                                         output_final_state=True, cu_seqlens=cu, state_indices=idx)
    assert st.data_ptr() == pool.data_ptr()
    outs = []
    for t in range(Tp, Tp + Td):
        o, _ = gdn.fused_recurrent_gated_delta_rule(g.q[:, t:t + 1], g.k[:, t:t + 1], g.v[:, t:t + 1], g.g[:, t:t + 1],
                                                    g.beta[:, t:t + 1], initial_state=pool, state_indices=idx)
        outs.append(o)
    o_ref, s_ref = C.recurrent(inp.q, inp.k, inp.v, inp.g, inp.beta, inp.scale)
    check_o(O, o_p.reshape(N, Tp, Hv, d), o_ref[:, :Tp])
    check_o(O, torch.cat(outs, 1), o_ref[:, Tp:])
    check_s(O, pool[idx.long()], s_ref)


def test_decode_layer_step_matches_separate_kernels_and_checker(gdn, checker):
    """The fused decode step of a whole layer (conv update + SiLU, q/k L2 norm, gate/beta, delta-rule update, gated norm
    in one kernel) over three chained steps with shared slot pools: states and convolution histories bit-identical to the
    separate kernels run one after the other (same rounding points), outputs equal to a bf16 rounding, and everything
    within the parity gates of the fp64 checker's composition."""
    O, C = checker
    N, Hk, Hv, d, W, slots = 6, 2, 4, 128, 4, 9
    Cn, cols = 2 * Hk * d + Hv * d, 2 * Hk * d + 2 * Hv * d + 2 * Hv
    gen = torch.Generator().manual_seed(17)
    conv_w = (torch.randn(Cn, W, generator=gen) / 2).bfloat16()
    A_log, dt_bias = torch.rand(Hv, generator=gen) * 2.77, 0.1 * torch.randn(Hv, generator=gen)
    norm_w = 1.0 + 0.1 * torch.randn(d, generator=gen)
    idx = torch.tensor([3, -1, 0, 7, 5, 8], dtype=torch.int32)
    pool0 = 0.02 * torch.randn(slots, Hv, d, d, generator=gen)
    conv0 = torch.randn(slots, W - 1, Cn, generator=gen).bfloat16()
    pool_f, pool_s, conv_f, conv_s = pool0.cuda(), pool0.cuda(), conv0.cuda(), conv0.cuda()
    pool_ref, conv_ref = pool0.double(), conv0.double()
    cw, Al, dtb, nw, ix = conv_w.cuda(), A_log.cuda(), dt_bias.cuda(), norm_w.cuda(), idx.cuda()
    for step in range(3):
        proj = torch.randn(N, cols + 8, generator=gen)
        proj[:, cols - 2 * Hv:cols] *= 2.0  # b and a drive sigmoid and softplus: give them range
        proj = proj.bfloat16()
        pg = proj.cuda()[:, :cols]  # a column slice of a wider projection output
        o_f = gdn.decode_layer_step(pg, cw, conv_f, Al, dtb, pool_f, ix, Hk=Hk, Hv=Hv, norm_weight=nw)
        # the same step from the separate entry points
        qkv = gdn.causal_conv1d_update(pg[:, :Cn], conv_s, cw, state_indices=ix)
        q = qkv[:, :Hk * d].reshape(N, 1, Hk, d)
        k = qkv[:, Hk * d:2 * Hk * d].reshape(N, 1, Hk, d)
        v = qkv[:, 2 * Hk * d:].reshape(N, 1, Hv, d)
        z = pg[:, Cn:Cn + Hv * d].reshape(N, 1, Hv, d)
        g, beta = gdn.gate_beta(pg[:, cols - Hv:cols], pg[:, cols - 2 * Hv:cols - Hv], Al, dtb)
        o_s, _ = gdn.fused_recurrent_gated_delta_rule(q, k, v, g.reshape(N, 1, Hv), beta.reshape(N, 1, Hv), initial_state=pool_s,
                                                      state_indices=ix, use_qk_l2norm_in_kernel=True, z=z, norm_weight=nw)
        assert gdn.read_status() == 0
        assert torch.equal(conv_f, conv_s), "conv history differs"
        assert torch.equal(pool_f, pool_s), f"state differs by {(pool_f - pool_s).abs().max().item():.3e}"
        # the two kernels may contract the output expression into different FMAs: outputs agree to a bf16 rounding
        e_sep = O.rel_l2(o_f.float().cpu(), o_s.reshape(N, Hv, d).float().cpu())
        assert e_sep <= 1e-3, f"output differs from the separate kernels: rel-L2 {e_sep:.3e}"
        assert torch.count_nonzero(o_f[1]) == 0
        # the checker's composition, sequence by sequence
        for n in range(N):
            sl = int(idx[n])
            if sl < 0:
                continue
            x = proj[n:n + 1, :cols].double()
            hist = torch.cat([conv_ref[sl], x[:, :Cn]], 0)[None]                    # [1, W, Cn]
            y = O.causal_conv1d_silu(hist, conv_w)[:, -1].to(torch.bfloat16).double()  # rounded where the device rounds
            conv_ref[sl] = hist[0, 1:]
            qr = O.l2norm(y[:, :Hk * d].reshape(1, 1, Hk, d))
            kr = O.l2norm(y[:, Hk * d:2 * Hk * d].reshape(1, 1, Hk, d))
            vr = y[:, 2 * Hk * d:].reshape(1, 1, Hv, d)
            zr = x[:, Cn:Cn + Hv * d].reshape(1, 1, Hv, d)
            gr, br = O.gate_beta(x[:, cols - Hv:cols], x[:, cols - 2 * Hv:cols - Hv], A_log, dt_bias)
            o_r, s_r = O.naive_recurrent_gated_delta_rule(qr, kr, vr, gr.float().double().reshape(1, 1, Hv), br.float().double().reshape(1, 1, Hv),
                                                          d ** -0.5, pool_ref[sl:sl + 1])
            pool_ref[sl] = s_r[0]
            y_r = O.gated_rmsnorm(o_r, zr, norm_w)
            assert O.rel_l2(o_f[n].float().cpu(), y_r[0, 0].to(torch.bfloat16).float()) <= 1e-3, (step, n)
            assert O.rel_l2(pool_f[sl].cpu(), s_r[0]) <= 1e-4, (step, n)
    assert torch.equal(conv_f.cpu().double(), conv_ref)
    # an index beyond the pools: skipped and flagged
    bad = torch.tensor([3, 99, 0, 7, 5, 8], dtype=torch.int32, device="cuda")
    before = pool_f.clone()
    o_b = gdn.decode_layer_step(pg, cw, conv_f, Al, dtb, pool_f, bad, Hk=Hk, Hv=Hv, norm_weight=nw)
    assert gdn.read_status() & 1 and torch.count_nonzero(o_b[1]) == 0
    untouched = [s for s in range(slots) if s not in (3, 0, 7, 5, 8)]
    assert torch.equal(pool_f[untouched], before[untouched])
