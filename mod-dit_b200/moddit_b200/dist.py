"""Ulysses-style re-sharding around the head-parallel hot path: sequence shards in, head shards inside.

Every stage of the path is independent per attention head, so P ranks each take H/P heads.  A caller
that holds sequence shards (1, H, N/P, D) exchanges them for head shards (1, H/P, N, D) with one
all-to-all per tensor before the path and one for the output after it.  The reference only has dead
hooks for this exchange (MoD/models/cogvideox/attention_processor.py:138-155, 220-229).

The functions take any initialised `torch.distributed` process group (NCCL on GPUs, gloo in CPU tests).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


def shard_bounds(total: int, world: int, rank: int):
    """[begin, end) of `rank`'s equal share; `total` must divide evenly."""
    if total % world:
        raise ValueError(f"{total} does not divide evenly over {world} ranks")
    per = total // world
    return rank * per, (rank + 1) * per


def seq_to_head(x: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """(1, H, N/P, D) sequence shard -> (1, H/P, N, D) head shard (heads [rank*H/P, (rank+1)*H/P))."""
    world = dist.get_world_size(group)
    if world == 1:
        return x
    _, H, ns, D = x.shape
    if H % world:
        raise ValueError(f"{H} heads do not divide over {world} ranks")
    hp = H // world
    send = x.reshape(world, hp, ns, D).contiguous()            # chunk p = heads of rank p
    recv = torch.empty_like(send)                              # chunk r = my heads, sequence shard of rank r
    dist.all_to_all_single(recv, send, group=group)
    return recv.permute(1, 0, 2, 3).reshape(1, hp, world * ns, D).contiguous()


def head_to_seq(x: torch.Tensor, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """(1, H/P, N, D) head shard -> (1, H, N/P, D) sequence shard."""
    world = dist.get_world_size(group)
    if world == 1:
        return x
    _, hp, N, D = x.shape
    if N % world:
        raise ValueError(f"sequence length {N} does not divide over {world} ranks")
    ns = N // world
    send = x.reshape(hp, world, ns, D).permute(1, 0, 2, 3).contiguous()   # chunk p = sequence shard of rank p
    recv = torch.empty_like(send)                                        # chunk r = heads of rank r
    dist.all_to_all_single(recv, send, group=group)
    return recv.reshape(1, world * hp, ns, D)
