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


def _failing_worker(rank, world, port, ret, scenario):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    launched = False
    try:
        if scenario == "raise_before_launch":
            # rank 1's preparation raises; it still answers the hand-shake, with ok=False, and every
            # rank learns of it on the host before anything is launched
            ok = True
            try:
                if rank == 1:
                    raise ValueError("mask construction failed on this rank")
            except ValueError:
                ok = False
            try:
                sharding.agree_to_launch(ok, timeout_s=20.0)
                launched = True
            except sharding.ShardingError as e:
                ret[rank] = ("refused", str(e))
        elif scenario == "absent_from_handshake":
            # rank 1 never joins: rank 0's hand-shake gives up after its host timeout
            if rank == 0:
                try:
                    sharding.agree_to_launch(True, timeout_s=2.0)
                    launched = True
                except sharding.ShardingError as e:
                    ret[rank] = ("refused", str(e))
            else:
                ret[rank] = ("absent", "")
        elif scenario == "skips_the_gather":
            # both ranks run their (stand-in) forward; rank 1 then skips the optional gather
            sharding.agree_to_launch(True, timeout_s=20.0)
            local = torch.full((1, 1, 128, 64), float(rank))
            if rank == 0:
                try:
                    sharding.all_gather_outputs(local, world, timeout_s=2.0)
                    ret[rank] = ("gathered", "")
                except sharding.ShardingError as e:
                    ret[rank] = ("gave_up", str(e))
            else:
                ret[rank] = ("skipped", "")
        assert not launched or scenario == "skips_the_gather"
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


@pytest.mark.parametrize("scenario,expect", [
    ("raise_before_launch", {0: "refused", 1: "refused"}),
    ("absent_from_handshake", {0: "refused", 1: "absent"}),
    ("skips_the_gather", {0: "gave_up", 1: "skipped"}),
])
def test_host_side_failures_between_ranks(scenario, expect):
    """A rank that fails before launch, one that never shows up, and one that skips the optional
    gather: the others find out on the host (a hand-shake on CPU tensors, a gather with a host
    timeout), raise ShardingError and launch nothing. No GPU is involved."""
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_failing_worker, args=(world, _free_port(), ret, scenario), nprocs=world, join=True)
    assert {k: v[0] for k, v in dict(ret).items()} == expect
    if scenario == "raise_before_launch":
        assert "reported a failure" in ret[0][1] and "this rank failed" in ret[1][1]
