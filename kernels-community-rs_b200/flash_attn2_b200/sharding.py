"""Multi-GPU partitioning of the attention path. One process per GPU; the units ((batch, head)
pairs, or whole packed sequences) are independent, so there is no collective on the data path.
torch.distributed (NCCL on GPUs, gloo in the CPU tests) is used only to gather shard outputs for
verification. The reference is single-GPU (its ops take the device from `q`), so these helpers
have no counterpart there.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_range(n_units: int, world: int, rank: int) -> range:
    """Contiguous, balanced split of n_units over `world` ranks (first ranks get the remainder)."""
    base, rem = divmod(n_units, world)
    start = rank * base + min(rank, rem)
    return range(start, start + base + (1 if rank < rem else 0))


def shard_heads(heads: int, heads_k: int, world: int, rank: int):
    """(query-head slice, kv-head slice) for a head split that keeps whole GQA groups together."""
    if heads % heads_k:
        raise ValueError("heads must be a multiple of heads_k")
    group = heads // heads_k
    r = shard_range(heads_k, world, rank)
    return slice(r.start * group, r.stop * group), slice(r.start, r.stop)


def shard_sequences_by_cost(lengths, world: int):
    """Greedy longest-first assignment of packed sequences to ranks by causal cost L^2.

    Returns one sorted list of sequence indices per rank."""
    order = sorted(range(len(lengths)), key=lambda i: -int(lengths[i]) ** 2)
    load = [0] * world
    out = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda j: (load[j], j))
        out[r].append(i)
        load[r] += int(lengths[i]) ** 2
    return [sorted(x) for x in out]


def pack_sequences(tensors, indices):
    """Concatenates the chosen sequences (list of [L_i, H, D]) and returns (packed, cu_seqlens)."""
    parts = [tensors[i] for i in indices]
    cu = [0]
    for p in parts:
        cu.append(cu[-1] + p.shape[0])
    if not parts:
        raise ValueError("a rank received no sequence")
    return torch.cat(parts, 0), torch.tensor(cu, dtype=torch.int32)


def gather_shards(local: torch.Tensor, dim: int, group=None) -> torch.Tensor:
    """All-gathers equally shaped shards and concatenates them along `dim` (verification only)."""
    world = dist.get_world_size(group)
    parts = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(parts, local.contiguous(), group=group)
    return torch.cat(parts, dim)
