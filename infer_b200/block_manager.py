"""Page allocator with prefix sharing for the paged KV pool.

Observable behaviour follows the reference's ``BlockManager``
(infer/engine/block_mannager.py:44-133): pages are handed out from the front of a
FIFO free list, a full page is keyed by the xxh64 digest of (digest of the previous
page, little-endian int64 token bytes), a second request whose leading pages carry
the same digests and token ids re-uses those physical pages and bumps their
reference counts, and a page returns to the back of the free list when its count
reaches zero.  The page ids this class returns for a given call sequence are
therefore the ones the reference returns; ``tests/golden`` pins that.

The attention kernels never see this class: they see the ``block_table`` lists it
fills in (through ``infer_b200.metadata``).
"""
from __future__ import annotations

from collections import deque

import numpy as np
import xxhash

from .sequence import Sequence

NO_HASH = -1


class Block:
    """One physical page: id, reference count, content digest."""

    __slots__ = ("block_id", "ref_count", "hash", "token_ids")

    def __init__(self, block_id: int):
        self.block_id = block_id
        self.ref_count = 0
        self.hash = NO_HASH
        self.token_ids: list[int] = []

    def update(self, digest: int, token_ids):
        self.hash = digest
        self.token_ids = token_ids

    def reset(self):
        self.ref_count = 1
        self.hash = NO_HASH
        self.token_ids = []


class BlockManager:
    def __init__(self, num_blocks: int, block_size: int):
        if num_blocks <= 0:
            raise ValueError("num_blocks must be positive")
        self.block_size = block_size
        self.blocks = [Block(i) for i in range(num_blocks)]
        self.hash_to_block_id: dict[int, int] = {}
        self.free_block_ids: deque[int] = deque(range(num_blocks))
        self.used_block_ids: set[int] = set()

    # -- digest chain (infer/engine/block_mannager.py:54-60) -------------------
    @staticmethod
    def compute_hash(token_ids, prefix: int = NO_HASH) -> int:
        state = xxhash.xxh64()
        if prefix != NO_HASH:
            state.update(int(prefix).to_bytes(8, "little"))
        state.update(np.asarray(token_ids, dtype=np.int64).tobytes())
        return state.intdigest()

    # -- free list -------------------------------------------------------------
    def _take(self, block_id: int) -> Block:
        page = self.blocks[block_id]
        if page.ref_count != 0:
            raise RuntimeError(f"page {block_id} is still referenced")
        page.reset()
        self.free_block_ids.remove(block_id)
        self.used_block_ids.add(block_id)
        return page

    def _give_back(self, block_id: int):
        if self.blocks[block_id].ref_count != 0:
            raise RuntimeError(f"page {block_id} is still referenced")
        self.used_block_ids.discard(block_id)
        self.free_block_ids.append(block_id)

    # -- whole-prompt allocation (infer/engine/block_mannager.py:76-103) -------
    def can_allocate(self, seq: Sequence) -> bool:
        return len(self.free_block_ids) >= seq.num_blocks

    def allocate(self, seq: Sequence):
        if seq.block_table:
            raise RuntimeError("sequence already has pages")
        digest = NO_HASH
        missed = False
        for i in range(seq.num_blocks):
            tokens = seq.block(i)
            full = len(tokens) == self.block_size
            digest = self.compute_hash(tokens, digest) if full else NO_HASH
            hit = self.hash_to_block_id.get(digest, -1)
            if hit == -1 or self.blocks[hit].token_ids != tokens:
                missed = True          # once one page misses, all later ones are fresh
            if missed:
                hit = self.free_block_ids[0]
                page = self._take(hit)
            else:
                seq.num_cached_tokens += self.block_size
                if hit in self.used_block_ids:
                    page = self.blocks[hit]
                    page.ref_count += 1
                else:                  # digest survived a free: revive the page
                    page = self._take(hit)
            if digest != NO_HASH:
                page.update(digest, tokens)
                self.hash_to_block_id[digest] = hit
            seq.block_table.append(hit)

    def deallocate(self, seq: Sequence):
        for block_id in reversed(seq.block_table):
            page = self.blocks[block_id]
            page.ref_count -= 1
            if page.ref_count == 0:
                self._give_back(block_id)
        seq.num_cached_tokens = 0
        seq.block_table.clear()

    # -- one-token growth (infer/engine/block_mannager.py:114-133) -------------
    def can_append(self, seq: Sequence) -> bool:
        return len(self.free_block_ids) >= (len(seq) % self.block_size == 1)

    def may_append(self, seq: Sequence):
        table = seq.block_table
        tail = self.blocks[table[-1]]
        rem = len(seq) % self.block_size
        if rem == 1:                   # first token of a new page
            if tail.hash == NO_HASH:
                raise RuntimeError("previous page was never sealed")
            fresh = self.free_block_ids[0]
            self._take(fresh)
            table.append(fresh)
        elif rem == 0:                 # page just filled: seal it with its digest
            if tail.hash != NO_HASH:
                raise RuntimeError("page sealed twice")
            tokens = seq.block(seq.num_blocks - 1)
            prev = self.blocks[table[-2]].hash if len(table) > 1 else NO_HASH
            digest = self.compute_hash(tokens, prev)
            tail.update(digest, tokens)
            self.hash_to_block_id[digest] = tail.block_id
        elif tail.hash != NO_HASH:
            raise RuntimeError("open page carries a digest")

    # -- accounting ------------------------------------------------------------
    def ref_counts(self) -> list[int]:
        return [b.ref_count for b in self.blocks]
