"""Seeded synthetic workloads with the shapes of the five benchmark configurations.

Integer metadata (context lengths, page lists, slots) always comes from a numpy
generator on the host, so it is identical wherever the workload is built.  Tensors come
from a ``torch.Generator`` on the requested device: parity tests build them on the CPU
and copy them to the GPU (oracle and kernel see the same bits); the benchmark builds
full-size pools directly on the GPU.

Page lists are produced the way the reference's engine produces them
(``BlockManager.allocate`` / ``may_append`` over ``Sequence`` objects,
infer/engine/block_mannager.py:79-133), on a shuffled free list so that the pages of a
sequence are scattered over the pool.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import numpy as np
import torch

from .block_manager import BlockManager
from .metadata import chunk_slots
from .sequence import Sequence

HEAD_DIM = 128
BLOCK_SIZE = 256


@dataclass
class Workload:
    name: str
    kind: str                       # "decode" | "prefill"
    n_q_heads: int
    n_kv_heads: int
    num_blocks: int
    block_tables: list              # list[list[int]], one page list per sequence
    context_lens: list              # keys per sequence, counting the appended tokens
    new_lens: list                  # tokens appended this step per sequence (1 for decode)
    slot_mapping: torch.Tensor      # int32 [sum(new_lens)]
    q: torch.Tensor                 # [sum(new_lens), Hq, d]
    k: torch.Tensor                 # [sum(new_lens), Hkv, d]
    v: torch.Tensor
    k_cache: torch.Tensor           # [num_blocks, block_size, Hkv, d] pre-filled
    v_cache: torch.Tensor
    fp8: bool = False
    head_dim: int = HEAD_DIM
    block_size: int = BLOCK_SIZE
    ref_counts: list = field(default_factory=list)
    scale: float = 1.0 / math.sqrt(HEAD_DIM)

    @property
    def batch(self):
        return len(self.context_lens)

    def block_tables_tensor(self, width=None):
        width = max(len(t) for t in self.block_tables) if width is None else width
        rows = [t + [-1] * (width - len(t)) for t in self.block_tables]
        return torch.tensor(rows, dtype=torch.int32)

    def context_lens_tensor(self):
        return torch.tensor(self.context_lens, dtype=torch.int32)

    def cu_seqlens(self):
        cu_q = np.concatenate([[0], np.cumsum(self.new_lens)]).astype(np.int32)
        cu_k = np.concatenate([[0], np.cumsum(self.context_lens)]).astype(np.int32)
        return torch.from_numpy(cu_q), torch.from_numpy(cu_k)

    def kv_bytes(self, elem_bytes=2, unique=True):
        """Algorithmic KV bytes one attention pass reads: tokens used in each page that
        is touched, K and V, all local heads; shared pages counted once if ``unique``."""
        per_token = self.n_kv_heads * self.head_dim * 2 * elem_bytes
        if not unique:
            return sum(self.context_lens) * per_token
        used = {}
        for table, n in zip(self.block_tables, self.context_lens):
            for i in range(-(-n // self.block_size)):
                fill = min(self.block_size, n - i * self.block_size)
                used[table[i]] = max(used.get(table[i], 0), fill)
        return sum(used.values()) * per_token

    def shard(self, rank: int, world: int) -> "Workload":
        """KV-head shard ``rank`` of ``world``: local pools, q/k/v and out keep only this
        rank's KV heads and their query heads; all integer metadata is replicated."""
        assert self.n_kv_heads % world == 0
        hk = self.n_kv_heads // world
        hq = self.n_q_heads // world
        ks, qs = slice(rank * hk, (rank + 1) * hk), slice(rank * hq, (rank + 1) * hq)
        import dataclasses
        return dataclasses.replace(
            self, n_q_heads=hq, n_kv_heads=hk,
            q=self.q[:, qs].contiguous(), k=self.k[:, ks].contiguous(), v=self.v[:, ks].contiguous(),
            k_cache=self.k_cache[:, :, ks].contiguous(), v_cache=self.v_cache[:, :, ks].contiguous())


def _randn(shape, gen, device, dtype=torch.bfloat16):
    return torch.randn(shape, generator=gen, device=device, dtype=torch.float32).to(dtype)


def _fill_pool(num_blocks, n_kv_heads, gen, device, dtype=torch.bfloat16):
    """N(0,1) pool, generated page-group by page-group to bound the fp32 temporary."""
    pool = torch.empty(num_blocks, BLOCK_SIZE, n_kv_heads, HEAD_DIM, device=device, dtype=dtype)
    step = 64
    for lo in range(0, num_blocks, step):
        hi = min(num_blocks, lo + step)
        pool[lo:hi] = _randn((hi - lo, BLOCK_SIZE, n_kv_heads, HEAD_DIM), gen, device, dtype)
    return pool


def _allocate(lens, num_blocks, rng, shared_prefix=0, n_shared=0):
    """Page lists for sequences of the given lengths via the engine's allocator.
    The first ``n_shared`` sequences start with the same ``shared_prefix`` token ids and
    so share those physical pages."""
    mgr = BlockManager(num_blocks, BLOCK_SIZE)
    mgr.free_block_ids = [int(i) for i in rng.permutation(num_blocks)]
    common = rng.integers(0, 32000, size=shared_prefix).tolist()
    tables = []
    for i, n in enumerate(lens):
        body = rng.integers(0, 32000, size=n - 1).tolist()
        if i < n_shared:
            body[:shared_prefix] = common
        seq = Sequence(body)
        mgr.allocate(seq)
        seq.append_token(int(rng.integers(0, 32000)))
        mgr.may_append(seq)
        tables.append(list(seq.block_table))
    return tables, mgr.ref_counts()


def _pool_size(lens, slack=1.1):
    pages = sum(-(-n // BLOCK_SIZE) for n in lens)
    return max(pages, math.ceil(slack * sum(lens) / BLOCK_SIZE))


def _decode_workload(name, seed, n_q_heads, n_kv_heads, lens, num_blocks, device,
                     shared_prefix=0, n_shared=0, fp8=False, with_pool=True, tensor_seed=None):
    rng = np.random.default_rng(seed)
    tables, refs = _allocate(lens, num_blocks, rng, shared_prefix, n_shared)
    slots = [t[(n - 1) // BLOCK_SIZE] * BLOCK_SIZE + (n - 1) % BLOCK_SIZE for t, n in zip(tables, lens)]
    gen = torch.Generator(device=device).manual_seed(seed if tensor_seed is None else tensor_seed)
    b = len(lens)
    q = _randn((b, n_q_heads, HEAD_DIM), gen, device)
    k = _randn((b, n_kv_heads, HEAD_DIM), gen, device)
    v = _randn((b, n_kv_heads, HEAD_DIM), gen, device)
    if with_pool:
        k_cache = _fill_pool(num_blocks, n_kv_heads, gen, device)
        v_cache = _fill_pool(num_blocks, n_kv_heads, gen, device)
    else:
        k_cache = v_cache = torch.empty(0)
    return Workload(name, "decode", n_q_heads, n_kv_heads, num_blocks, tables, list(map(int, lens)),
                    [1] * b, torch.tensor(slots, dtype=torch.int32), q, k, v, k_cache, v_cache,
                    fp8=fp8, ref_counts=refs)


def config0(device="cpu", seed=1000):
    """Qwen3-0.6B-shaped layer: Hq16/Hkv8, 64-page pool, 8 sequences, ctx U{64..1024}."""
    rng = np.random.default_rng(seed)
    lens = rng.integers(64, 1025, size=8)
    return _decode_workload("qwen3-0.6b-decode", seed, 16, 8, lens, 64, device)


def config1(device="cpu", seed=1001, batch=64, lo=512, hi=8192, n_kv_heads=8, n_q_heads=32,
            with_pool=True, tensor_seed=None):
    """Qwen3-8B decode shape: Hq32/Hkv8, 64 sequences, ctx U{512..8192}, pool = tokens + 10%.
    ``n_kv_heads``/``n_q_heads`` below 8/32 build one KV-head shard directly; ``tensor_seed``
    then gives each shard its own values while the integer metadata stays replicated."""
    rng = np.random.default_rng(seed)
    lens = rng.integers(lo, hi + 1, size=batch)
    return _decode_workload("qwen3-8b-decode", seed, n_q_heads, n_kv_heads, lens, _pool_size(lens),
                            device, with_pool=with_pool, tensor_seed=tensor_seed)


def config2(device="cpu", seed=1002, n_seqs=16, max_prefix=4096, chunk=2048):
    """Paged chunked prefill: Hq16/Hkv8, cached prefix U{0..max_prefix}, new chunk appended
    through slot_mapping, causal attention over prefix + chunk."""
    rng = np.random.default_rng(seed)
    prefixes = rng.integers(0, max_prefix + 1, size=n_seqs)
    lens = [int(p) + chunk for p in prefixes]
    num_blocks = _pool_size(lens)
    perm = [int(i) for i in rng.permutation(num_blocks)]
    tables, at = [], 0
    for n in lens:
        need = -(-n // BLOCK_SIZE)
        tables.append(perm[at:at + need])
        at += need
    slots = []
    for t, p, n in zip(tables, prefixes, lens):
        slots.extend(chunk_slots(t, int(p), n, BLOCK_SIZE))
    gen = torch.Generator(device=device).manual_seed(seed)
    total_q = n_seqs * chunk
    q = _randn((total_q, 16, HEAD_DIM), gen, device)
    k = _randn((total_q, 8, HEAD_DIM), gen, device)
    v = _randn((total_q, 8, HEAD_DIM), gen, device)
    k_cache = _fill_pool(num_blocks, 8, gen, device)
    v_cache = _fill_pool(num_blocks, 8, gen, device)
    return Workload("chunked-prefill", "prefill", 16, 8, num_blocks, tables, lens, [chunk] * n_seqs,
                    torch.tensor(slots, dtype=torch.int32), q, k, v, k_cache, v_cache)


def config3(device="cpu", seed=1003):
    """FP8 KV on config0's shapes; 1% of k entries are multiplied by 20.  The pools hold
    bf16 source data here; the FP8 pool is built from them by appending page by page."""
    w = config0(device, seed)
    gen = torch.Generator(device=device).manual_seed(seed + 7)
    for t in (w.k, w.k_cache):
        spike = torch.rand(t.shape, generator=gen, device=device) < 0.01
        t[spike] = (t[spike].float() * 20).to(t.dtype)
    w.name, w.fp8 = "fp8-kv-decode", True
    return w


def config4(device="cpu", seed=1004, batch=256, cap=32768, with_pool=True, n_kv_heads=8, n_q_heads=64,
            tensor_seed=None, longest_at_cap=False):
    """Qwen3-32B long-context shape: Hq64/Hkv8, ctx lognormal(median 4096, sigma 0.8) capped
    at 32768; the first half of the batch shares the pages of a 2048-token prefix.
    ``n_kv_heads``/``n_q_heads`` below 8/64 build one KV-head shard directly (see config1)."""
    rng = np.random.default_rng(seed)
    lens = np.minimum(cap, np.floor(rng.lognormal(math.log(4096), 0.8, size=batch))).astype(np.int64)
    n_shared = batch // 2
    lens[:n_shared] = np.maximum(lens[:n_shared], 2049)
    lens = np.maximum(lens, 2)
    if longest_at_cap:            # tests: make sure one context really is `cap` tokens long (the draw's maximum may fall short)
        lens[int(np.argmax(lens))] = cap
    pages = sum(-(-int(n) // BLOCK_SIZE) for n in lens)
    num_blocks = max(pages, math.ceil(1.1 * int(lens.sum()) / BLOCK_SIZE))
    return _decode_workload("qwen3-32b-long-decode", seed, n_q_heads, n_kv_heads, lens, num_blocks, device,
                            shared_prefix=2048, n_shared=n_shared, with_pool=with_pool, tensor_seed=tensor_seed)


CONFIGS = [config0, config1, config2, config3, config4]
