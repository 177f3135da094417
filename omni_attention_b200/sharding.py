"""Multi-GPU use: shard the flattened (batch * head) axis across ranks.

Every (batch, head) pair is an independent attention problem with its own rows of the block lists
(the reference's grid is (num_q_blocks, B*H), omni-attn-mma/mma/omni_attn_shared_kv.cu:789-790), so
ranks never exchange anything on the data path. The only collective offered is an optional
all-gather of the outputs for callers that want the full tensor on every rank.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
from torch import Tensor

from .block_mask import OmniBlockMask


def shard_range(total_bh: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous range of (batch*head) pairs owned by ``rank``: sizes differ by at most one."""
    base, rem = divmod(total_bh, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def balanced_shard_ranges(work_per_bh: Tensor, world: int) -> List[Tuple[int, int]]:
    """Contiguous ranges whose summed work (e.g. visited blocks per pair) is as close to even as a greedy
    prefix split gets (a pair joins the current rank while that brings the running total closer to the
    rank's target); every rank gets at least one pair when there are enough pairs."""
    n = int(work_per_bh.numel())
    w = work_per_bh.double().flatten()
    total = float(w.sum())
    bounds, acc, start = [], 0.0, 0
    for r in range(world):
        if r == world - 1:
            end = n
        else:
            target = total * (r + 1) / world
            end = start
            while end < n - (world - 1 - r) and (end == start or abs(acc + float(w[end]) - target) <= abs(acc - target)):
                acc += float(w[end])
                end += 1
        bounds.append((start, end))
        start = end
    return bounds


def shard_block_mask(bm: OmniBlockMask, rank: int, world: int) -> Tuple[OmniBlockMask, Tuple[int, int]]:
    B, H, _ = bm.kv_num_blocks.shape
    lo, hi = shard_range(B * H, rank, world)
    return bm.slice_heads(lo, hi), (lo, hi)


def shard_qkv(t: Tensor, rank: int, world: int) -> Tensor:
    """[B, H, N, D] -> [1, n_local, N, D] view of this rank's pairs."""
    B, H, N, D = t.shape
    lo, hi = shard_range(B * H, rank, world)
    return t.reshape(B * H, N, D)[lo:hi].unsqueeze(0)


class ShardingError(RuntimeError):
    """A peer rank reported a failure, or did not show up for a host-side hand-shake or the gather in time."""


def agree_to_launch(ok: bool, group=None, timeout_s: float = 30.0) -> None:
    """Host-side hand-shake before a sharded step: every rank says whether it is ready to launch
    (``ok=False`` from a rank whose own preparation raised). Returns when all ranks are; raises
    ShardingError on every rank when any rank is not, or when a rank does not answer within
    ``timeout_s``, so that no rank launches work whose result nobody will collect. Runs on CPU tensors
    (use a gloo group next to the NCCL one on GPUs): the ranks learn of a failure on the host, with
    none of their kernels or collectives in flight. The reference is single-GPU and has no
    counterpart; its whole error story is a cudaGetLastError after the launch
    (omni-attn-mma/mma/omni_attn_shared_kv.cu:1005-1008)."""
    import datetime

    import torch.distributed as dist

    flag = torch.tensor([1 if ok else 0], dtype=torch.int32)
    try:
        work = dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group, async_op=True)
        work.wait(timeout=datetime.timedelta(seconds=timeout_s))
    except Exception as e:  # a peer that never joins ends the wait with the backend's timeout error
        raise ShardingError(f"a rank did not answer the launch hand-shake within {timeout_s} s: {e}") from e
    if int(flag[0]) != 1:
        raise ShardingError("a rank reported a failure before launch" if ok else "this rank failed before launch")


def all_gather_outputs(local_out: Tensor, total_bh: int, group=None, timeout_s: Optional[float] = None) -> Tensor:
    """Optional epilogue: gather every rank's [1, n_local, N, D] output into [total_bh, N, D] on all
    ranks (NCCL on GPUs, gloo on CPU). Not part of the timed forward. With ``timeout_s`` the host gives
    up waiting after that many seconds and raises ShardingError (a rank that skipped the gather)."""
    import datetime

    import torch.distributed as dist

    world = dist.get_world_size(group)
    N, D = local_out.shape[2:]
    sizes = [shard_range(total_bh, r, world) for r in range(world)]
    parts = [torch.empty(hi - lo, N, D, dtype=local_out.dtype, device=local_out.device) for lo, hi in sizes]
    mine = local_out.reshape(-1, N, D).contiguous()
    if timeout_s is None:
        dist.all_gather(parts, mine, group=group)
    else:
        try:
            work = dist.all_gather(parts, mine, group=group, async_op=True)
            work.wait(timeout=datetime.timedelta(seconds=timeout_s))
        except Exception as e:
            raise ShardingError(f"all-gather of the outputs did not complete within {timeout_s} s: {e}") from e
    return torch.cat(parts, 0)


def max_over_ranks(value: float, device: Optional[torch.device] = None, group=None) -> float:
    """A time reported for a multi-GPU step is the slowest rank's."""
    import torch.distributed as dist

    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t[0])
