"""GPU tests of the fused all-gather: the gated-norm stage stores every output row into all given buffers."""
import os
import socket

import pytest
import torch

from avelang_b200 import synth

pytestmark = pytest.mark.gpu


def test_peer_scatter_single_gpu(built_lib):
    """Two buffers on one GPU stand in for two ranks: both must receive the rows, at the head slice's offsets."""
    from avelang_b200 import gdn
    inp = synth.make_inputs(2, 200, 2, 4, 128, 128, seed=3, with_z=True, gate_scale=0.1).to("cuda")
    ref, _ = gdn.chunk_gated_delta_rule(inp.q, inp.k, inp.v, inp.g, inp.beta, z=inp.z)
    # the local output is heads [4, 8) of a 12-head buffer
    bufs = [torch.zeros(2, 200, 12, 128, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    off = 4 * 128 * 2
    peers = torch.tensor([b.data_ptr() + off for b in bufs], dtype=torch.int64, device="cuda")
    gdn.chunk_gated_delta_rule(inp.q, inp.k, inp.v, inp.g, inp.beta, z=inp.z, out=bufs[0][:, :, 4:8], out_peers=peers)
    torch.cuda.synchronize()
    for b in bufs:
        assert torch.equal(b[:, :, 4:8], ref)
        assert torch.count_nonzero(b[:, :, :4]) == 0 and torch.count_nonzero(b[:, :, 8:]) == 0
    with pytest.raises(ValueError):
        gdn.chunk_gated_delta_rule(inp.q, inp.k, inp.v, inp.g, inp.beta, out_peers=peers)  # needs z


def _rank_main(rank, world, port, ret, B=2, T=200):
    import torch.distributed as dist
    from avelang_b200.block import GdnBlockShard
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        hidden, Hk, Hv, d = 256, 2, 4, 128
        g = torch.Generator().manual_seed(0)
        w_in = (0.02 * torch.randn(2 * Hk * d + 2 * Hv * d + 2 * Hv, hidden, generator=g)).bfloat16()
        conv_w = (torch.randn(2 * Hk * d + Hv * d, 4, generator=g) / 2).bfloat16()
        A_log, dt_bias = torch.rand(Hv, generator=g) * 2.77, 0.1 * torch.randn(Hv, generator=g)
        x = torch.randn(B, T, hidden, generator=g).bfloat16().cuda()
        blk = GdnBlockShard(w_in, conv_w, A_log, dt_bias, torch.ones(d), Hk=Hk, Hv=Hv, dk=d, dv=d, rank=rank, world=world)
        y_nccl = blk.forward(x)
        y_fused = blk.forward(x, fused_gather=True).clone()
        ret[rank] = bool(torch.equal(y_nccl, y_fused))
        ret[10 + rank] = float((y_fused.float() - y_nccl.float()).norm() / y_nccl.float().norm())
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_gather_matches_nccl_two_ranks(built_lib):
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_rank_main, args=(2, port, ret), nprocs=2, join=True)
    assert ret[0] is True and ret[1] is True


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_gather_close_to_nccl_when_schedules_differ(built_lib):
    """One long sequence and two value heads per rank: the NCCL path walks it as parallel parts, the fused path (whose
    norm kernel pushes rows range by range) as plain chains.  Each is within 1e-3 of the checker, so the two may differ
    by 2e-3 but no more."""
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_rank_main, args=(2, port, ret, 1, 4096), nprocs=2, join=True)
    assert ret[10] <= 2e-3 and ret[11] <= 2e-3, dict(ret)


def _rank_tp(rank, world, port, ret):
    """Row-parallel output projection on two ranks against the unsharded block on rank 0's GPU."""
    import torch.distributed as dist
    from avelang_b200.block import GdnBlockShard, GdnBlockTP
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        hidden, Hk, Hv, d, B, T = 256, 2, 4, 128, 1, 130
        g = torch.Generator().manual_seed(0)
        w_in = (0.02 * torch.randn(2 * Hk * d + 2 * Hv * d + 2 * Hv, hidden, generator=g)).bfloat16()
        conv_w = (torch.randn(2 * Hk * d + Hv * d, 4, generator=g) / 2).bfloat16()
        A_log, dt_bias = torch.rand(Hv, generator=g) * 2.77, 0.1 * torch.randn(Hv, generator=g)
        w_out = (0.05 * torch.randn(hidden, Hv * d, generator=g)).bfloat16()
        x = torch.randn(B, T, hidden, generator=g).bfloat16().cuda()
        tp = GdnBlockTP(w_in, conv_w, A_log, dt_bias, torch.ones(d), w_out, Hk=Hk, Hv=Hv, dk=d, dv=d, rank=rank, world=world,
                        device=f"cuda:{rank}")
        y = tp.forward(x)
        # the same projection with the sum fused into the GEMM (peer stores into the owners' staging slots), twice: the
        # second call reuses the buffers
        y_f = tp.forward(x, fused_reduce=True).clone()
        y_f2 = tp.forward(x, fused_reduce=True)
        heads = GdnBlockShard(w_in, conv_w, A_log, dt_bias, torch.ones(d), Hk=Hk, Hv=Hv, dk=d, dv=d, device=f"cuda:{rank}").forward(x)
        ref = heads.reshape(B * T, -1).float() @ w_out.cuda().float().T
        err = ((y.reshape(B * T, -1).float() - ref).norm() / ref.norm()).item()
        ret[rank] = err
        ret[10 + rank] = ((y_f.reshape(B * T, -1).float() - ref).norm() / ref.norm()).item()
        ret[20 + rank] = bool(torch.equal(y_f, y_f2))
        both = [torch.empty_like(y_f) for _ in range(world)]
        dist.all_gather(both, y_f.contiguous())
        ret[30 + rank] = bool(torch.equal(both[0], both[1]))  # every rank holds the same bits
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_row_parallel_output_projection_two_ranks(built_lib):
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_rank_tp, args=(2, port, ret), nprocs=2, join=True)
    r = dict(ret)
    assert r[0] < 1e-2 and r[1] < 1e-2, r              # NCCL all-reduce path vs the unsharded block
    assert r[10] < 1e-2 and r[11] < 1e-2, r            # sum fused into the GEMM
    assert r[20] and r[21] and r[30] and r[31], r      # repeatable, and the same bits on both ranks
