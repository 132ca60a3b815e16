"""Multi-GPU use of the path: one process per GPU.

Every (batch, head) pair is independent, so the default partition is by head with no data-path
collective.  When activations arrive sequence-sharded, the optional Ulysses mode turns them into
head shards with one all-to-all before the attention and one after it (NCCL over NVLink; gloo in
the CPU tests).  The permutation is over the whole sequence, so the exchange must come first.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch
import torch.distributed as dist


def head_range(n_heads: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous block of heads owned by `rank` (sizes differ by at most one)."""
    base, extra = divmod(n_heads, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def balanced_head_partition(kept_per_head: Sequence[int], world: int) -> List[List[int]]:
    """Longest-processing-time assignment of heads to ranks by kept-block count; used when
    densities differ strongly between heads.  Returns the head ids of each rank, ascending."""
    order = sorted(range(len(kept_per_head)), key=lambda h: (-int(kept_per_head[h]), h))
    loads = [0] * world
    parts: List[List[int]] = [[] for _ in range(world)]
    for h in order:
        r = min(range(world), key=lambda i: (loads[i], i))
        parts[r].append(h)
        loads[r] += int(kept_per_head[h])
    return [sorted(p) for p in parts]


def ulysses_seq_to_heads(x: torch.Tensor, group=None) -> torch.Tensor:
    """[B, H, N/P, D] on every rank (rank r holds token slice r) -> [B, H/P, N, D] (rank r holds
    head block r).  H must be divisible by the group size and all token slices equal."""
    world = dist.get_world_size(group)
    B, H, n_loc, D = x.shape
    if H % world:
        raise ValueError(f"{H} heads cannot be split over {world} ranks")
    send = x.reshape(B, world, H // world, n_loc, D).permute(1, 0, 2, 3, 4).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    # recv[s] = token slice s of my head block
    return recv.permute(1, 2, 0, 3, 4).reshape(B, H // world, world * n_loc, D)


def ulysses_heads_to_seq(x: torch.Tensor, group=None) -> torch.Tensor:
    """Inverse of `ulysses_seq_to_heads`: [B, H/P, N, D] -> [B, H, N/P, D]."""
    world = dist.get_world_size(group)
    B, h_loc, N, D = x.shape
    if N % world:
        raise ValueError(f"{N} tokens cannot be split over {world} ranks")
    n_loc = N // world
    send = x.reshape(B, h_loc, world, n_loc, D).permute(2, 0, 1, 3, 4).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    # recv[r] = my token slice of head block r
    return recv.permute(1, 0, 2, 3, 4).reshape(B, world * h_loc, n_loc, D)
