"""CPU tests of the multi-GPU host logic: head partitioning, projection-row selection, and the head all-gather
run as two gloo ranks."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from avelang_b200.block import HeadShard, gather_heads, output_projection_columns, projection_rows


def test_head_shards_partition_all_heads():
    for world in (1, 2, 4, 8):
        kh, vh = [], []
        for r in range(world):
            s = HeadShard(r, world, 16, 32)
            kh += list(s.key_heads)
            vh += list(s.value_heads)
            # every value head of the shard reads a key head of the same shard
            assert all(h // 2 in s.key_heads for h in s.value_heads)
        assert kh == list(range(16)) and vh == list(range(32))
    with pytest.raises(ValueError):
        HeadShard(0, 3, 16, 32)


def test_projection_rows_cover_weight_once():
    rows = torch.cat([projection_rows(HeadShard(r, 8, 16, 32), 128, 128) for r in range(8)])
    assert rows.numel() == 12352 and torch.equal(rows.sort().values, torch.arange(12352))
    assert projection_rows(HeadShard(3, 8, 16, 32), 128, 128).numel() == 1544


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = torch.arange(2 * 5 * 4 * 3, dtype=torch.float32).reshape(2, 5, 4, 3)
        hl = 4 // world
        local = full[:, :, rank * hl:(rank + 1) * hl].contiguous()
        got = gather_heads(local, world)
        out[rank] = bool(torch.equal(got, full))
    finally:
        dist.destroy_process_group()


def test_gather_heads_two_gloo_ranks():
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_rank_main, args=(2, _free_port(), out), nprocs=2, join=True)
    assert dict(out) == {0: True, 1: True}


def _rank_out_proj(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        Hv, dv, hidden = 4, 8, 16
        heads = torch.randn(6, Hv, dv, generator=g)
        w_out = torch.randn(hidden, Hv * dv, generator=g)
        shard = HeadShard(rank, world, 2, Hv)
        part = heads[:, shard.value_heads].reshape(6, -1) @ w_out[:, output_projection_columns(shard, dv)].T
        dist.all_reduce(part)
        out[rank] = bool(torch.allclose(part, heads.reshape(6, -1) @ w_out.T, atol=1e-5))
    finally:
        dist.destroy_process_group()


def test_row_parallel_output_projection_two_gloo_ranks():
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_rank_out_proj, args=(2, _free_port(), out), nprocs=2, join=True)
    assert dict(out) == {0: True, 1: True}
