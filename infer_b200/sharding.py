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


class PeerMissing(RuntimeError):
    """A rank did not reach a step within the time limit."""

    def __init__(self, step: int, ranks: list[int], waited_s: float):
        super().__init__(f"step {step}: rank(s) {ranks} did not arrive within {waited_s:.1f} s")
        self.step, self.ranks = step, ranks


class StepRendezvous:
    """Host-side check that every rank is still there before a step's collective is launched.

    The attention path has no exchange step, so a rank that died or hung is only noticed at the
    validation gather, where the survivors would block inside the collective.  Before a gather
    every rank writes ``step<N>/rank<r>`` into the process group's key-value store and waits
    (with a time limit) for its peers' keys; when the limit runs out it raises ``PeerMissing``
    naming the ranks whose key never appeared, with no collective in flight and no kernel
    launched.  Nothing here touches a GPU."""

    def __init__(self, store, rank: int, world: int, timeout_s: float = 30.0):
        self.store, self.rank, self.world, self.timeout_s = store, rank, world, timeout_s

    def arrive(self, step: int):
        import time
        from datetime import timedelta
        self.store.set(f"step{step}/rank{self.rank}", b"1")
        keys = [f"step{step}/rank{r}" for r in range(self.world) if r != self.rank]
        t0 = time.monotonic()
        try:
            if keys:
                self.store.wait(keys, timedelta(seconds=self.timeout_s))
        except Exception:
            missing = []
            for r in range(self.world):
                if r == self.rank:
                    continue
                try:
                    self.store.wait([f"step{step}/rank{r}"], timedelta(milliseconds=10))
                except Exception:
                    missing.append(r)
            raise PeerMissing(step, missing, time.monotonic() - t0) from None


def checked_gather_heads(local: torch.Tensor, rendezvous: StepRendezvous, step: int, group=None) -> torch.Tensor:
    """``gather_heads`` that first makes sure every rank reached this step."""
    rendezvous.arrive(step)
    return gather_heads(local, group)
