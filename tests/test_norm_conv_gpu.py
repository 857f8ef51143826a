"""GPU parity of the streaming helpers: gated RMSNorm, causal conv1d + SiLU, gate/beta math."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gdn(built_lib):
    from avelang_b200 import gdn
    return gdn


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("gate_first", [False, True])
def test_gated_rmsnorm(gdn, checker, d, gate_first):
    O, _ = checker
    g = torch.Generator().manual_seed(d)
    x = (torch.randn(3, 37, 5, d, generator=g) * 3).bfloat16()
    z = torch.randn(3, 37, 5, d, generator=g).bfloat16()
    w = torch.linspace(0.5, 2.0, d)
    y = gdn.gated_rmsnorm(x.cuda(), z.cuda(), w.cuda(), gate_first=gate_first)
    if gate_first:
        xz = x.double() * torch.nn.functional.silu(z.double())
        ref = xz * torch.rsqrt(xz.pow(2).mean(-1, keepdim=True) + 1e-6) * w.double()
    else:
        ref = O.gated_rmsnorm(x, z, w)
    assert O.rel_l2(y.float().cpu(), ref.bfloat16().float()) < 1e-3
    # strided input (a head slice) and out=
    out = torch.empty(3, 37, 2, d, dtype=torch.bfloat16, device="cuda")
    gdn.gated_rmsnorm(x.cuda()[:, :, 1:3], z.cuda()[:, :, 1:3], w.cuda(), gate_first=gate_first, out=out)
    assert torch.equal(out, y[:, :, 1:3])


def test_gated_rmsnorm_empty(gdn):
    x = torch.zeros(0, 4, 128, dtype=torch.bfloat16, device="cuda")
    assert gdn.gated_rmsnorm(x, x).shape == (0, 4, 128)


@pytest.mark.parametrize("width", [2, 3, 4])
def test_causal_conv1d_silu(gdn, checker, width):
    O, _ = checker
    g = torch.Generator().manual_seed(width)
    x = torch.randn(2, 150, 96, generator=g).bfloat16()
    w = (torch.randn(96, width, generator=g) / 2).bfloat16()
    bias = torch.randn(96, generator=g).bfloat16()
    y = gdn.causal_conv1d_silu(x.cuda(), w.cuda())
    assert O.rel_l2(y.float().cpu(), O.causal_conv1d_silu(x, w).bfloat16().float()) < 1e-3
    yb = gdn.causal_conv1d_silu(x.cuda(), w.cuda(), bias.cuda())
    ref = O.causal_conv1d_silu(x, w)  # bias enters before the SiLU: recompute by hand
    xs = x.double()
    acc = torch.zeros_like(xs)
    for j in range(width):
        sh = width - 1 - j
        acc[:, sh:] += xs[:, : xs.shape[1] - sh] * w.double()[:, j]
    acc = acc + bias.double()
    assert O.rel_l2(yb.float().cpu(), (acc * torch.sigmoid(acc)).bfloat16().float()) < 1e-3
    assert ref.shape == y.shape


def test_causal_conv1d_varlen_and_column_slice(gdn, checker):
    O, _ = checker
    g = torch.Generator().manual_seed(0)
    wide = torch.randn(1, 300, 160, generator=g).bfloat16()
    w = (torch.randn(64, 4, generator=g) / 2).bfloat16()
    cu = torch.tensor([0, 1, 3, 64, 65, 200, 300], dtype=torch.int32)
    x = wide[:, :, 32:96]  # a column slice of a wider tensor: row stride 160
    y = gdn.causal_conv1d_silu(x.cuda(), w.cuda(), cu_seqlens=cu.cuda())
    assert O.rel_l2(y.float().cpu(), O.causal_conv1d_silu(x, w, cu).bfloat16().float()) < 1e-3


def test_gate_beta(gdn, checker):
    O, _ = checker
    g = torch.Generator().manual_seed(0)
    wide = (torch.randn(500, 24, generator=g) * 3).bfloat16()
    A_log, dt_bias = torch.rand(8, generator=g) * 2.77, 0.1 * torch.randn(8, generator=g)
    a_in, b_in = wide[:, 16:24], wide[:, 8:16]
    gg, beta = gdn.gate_beta(a_in.cuda(), b_in.cuda(), A_log.cuda(), dt_bias.cuda())
    g_ref, beta_ref = O.gate_beta(a_in, b_in, A_log, dt_bias)
    assert O.rel_l2(gg.cpu(), g_ref) < 1e-5 and O.rel_l2(beta.cpu(), beta_ref) < 1e-5
    assert (gg <= 0).all()


def test_conv1d_update_matches_full_convolution(gdn, checker):
    """T single-token updates from an empty history reproduce the causal convolution over the T tokens."""
    O, _ = checker
    g = torch.Generator().manual_seed(1)
    N, T, Cn, W = 3, 9, 64, 4
    x = torch.randn(N, T, Cn, generator=g).bfloat16()
    w = (torch.randn(Cn, W, generator=g) / 2).bfloat16()
    state = torch.zeros(5, W - 1, Cn, dtype=torch.bfloat16, device="cuda")
    idx = torch.tensor([4, -1, 0], dtype=torch.int32, device="cuda")
    ys = [gdn.causal_conv1d_update(x[:, t].cuda(), state, w.cuda(), state_indices=idx) for t in range(T)]
    y = torch.stack(ys, 1)
    ref = O.causal_conv1d_silu(x, w).bfloat16().float()
    for n in (0, 2):
        assert O.rel_l2(y[n].float().cpu(), ref[n]) < 1e-3
    # the history now holds the last W-1 inputs, oldest first; untouched slots stay zero
    assert torch.equal(state[4].cpu(), x[0, T - (W - 1):]) and torch.equal(state[0].cpu(), x[2, T - (W - 1):])
    assert torch.count_nonzero(state[1:4]) == 0
    assert gdn.read_status() == 0  # a negative index is a request to skip, not an error
    # an index beyond the pool: that sequence is skipped (history and output row untouched) and the status word says so
    before = state.clone()
    y_prev = torch.full((N, Cn), 7.0, dtype=torch.bfloat16, device="cuda")
    bad = torch.tensor([4, 5, 0], dtype=torch.int32, device="cuda")
    gdn.causal_conv1d_update(x[:, 0].cuda(), state, w.cuda(), state_indices=bad, out=y_prev)
    assert gdn.read_status() & 1  # AVE_GDN_DEV_BAD_SLOT
    assert torch.equal(y_prev[1], torch.full((Cn,), 7.0, dtype=torch.bfloat16, device="cuda"))
    assert torch.equal(state[1:4], before[1:4])
