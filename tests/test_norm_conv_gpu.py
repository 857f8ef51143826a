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
