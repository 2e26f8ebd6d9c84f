"""KV-head sharding across GPUs (the Qwen3 tensor-parallel layout the reference's unused
``tensor_parallel_size`` field anticipates, infer/config.py:12,22).

Rank r of G owns kv heads [r*Hkv/G, (r+1)*Hkv/G) and their query heads: local pools, q, k, v
and outputs carry only those heads; page ids, slots and lengths are replicated.  The
attention path needs no exchange; ``gather_heads`` (an all_gather over the process group,
NCCL on GPUs) only reassembles outputs for validation."""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_bounds(n_heads: int, rank: int, world: int):
    if n_heads % world:
        raise ValueError(f"{n_heads} heads do not split over {world} ranks")
    per = n_heads // world
    return rank * per, (rank + 1) * per


def gather_heads(local: torch.Tensor, group=None) -> torch.Tensor:
    """[T, H/G, d] on every rank -> [T, H, d] on every rank."""
    world = dist.get_world_size(group)
    parts = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(parts, local.contiguous(), group=group)
    return torch.cat(parts, dim=1)
