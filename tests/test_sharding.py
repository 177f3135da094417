"""batch*head sharding: host logic, and a world_size-2 gloo run on CPU."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from omni_attention_b200 import inputs, sharding
from omni_attention_b200.block_mask import create_causal_omni_block_mask


def test_shard_ranges_cover_everything_once():
    for total in (1, 7, 8, 32, 128):
        for world in (1, 2, 3, 4, 8):
            if world > total:
                continue
            r = [sharding.shard_range(total, k, world) for k in range(world)]
            assert r[0][0] == 0 and r[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(r, r[1:]))
            sizes = [b - a for a, b in r]
            assert max(sizes) - min(sizes) <= 1


def test_balanced_ranges():
    w = torch.tensor([1, 1, 1, 1, 10, 10, 1, 1], dtype=torch.float64)
    r = sharding.balanced_shard_ranges(w, 2)
    assert r[0][0] == 0 and r[-1][1] == 8 and r[0][1] == r[1][0]
    s = [float(w[a:b].sum()) for a, b in r]
    assert max(s) <= 16
    r = sharding.balanced_shard_ranges(torch.ones(4), 4)
    assert r == [(0, 1), (1, 2), (2, 3), (3, 4)]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, H, N, D = 2, 3, 256, 64
        q, k, v = inputs.make_qkv(B, H, N, D, torch.float32, seed=1)
        bm = create_causal_omni_block_mask(B, H, N, N)
        shard, (lo, hi) = sharding.shard_block_mask(bm, rank, world)
        qs = sharding.shard_qkv(q, rank, world)
        # the same shard drawn directly must be identical (ranks generate only their own slice)
        qd, _, _ = inputs.make_qkv(B, H, N, D, torch.float32, seed=1, bh_range=(lo, hi))
        assert torch.equal(qs, qd)
        assert shard.kv_num_blocks.shape == (1, hi - lo, N // 128)
        # stand-in for the forward: each rank tags its rows; gather must restore global order
        local = qs * 0 + torch.arange(lo, hi, dtype=torch.float32).view(1, -1, 1, 1)
        full = sharding.all_gather_outputs(local, B * H)
        assert full.shape == (B * H, N, D)
        assert torch.equal(full[:, 0, 0], torch.arange(B * H, dtype=torch.float32))
        t = sharding.max_over_ranks(10.0 + rank)
        assert t == 10.0 + world - 1
        ret[rank] = 1
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_shard_and_gather():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    port = _free_port()
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert dict(ret) == {0: 1, 1: 1}
