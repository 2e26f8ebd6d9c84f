"""``BlockManager``: Python face of the native page allocator.

The allocator itself is C++ (include/block_manager.hpp, exported through the C ABI as
``infer_block_manager_*``); this class only keeps the call signatures the reference's
scheduler uses on its ``BlockManager`` (infer/engine/scheduler.py:27-61:
``can_allocate / allocate / can_append / may_append / deallocate`` taking a ``Sequence``)
and copies the resulting page list back into ``seq.block_table``.  Page ids, cache hits,
reference counts and free-list order equal the reference's for the same call sequence
(pinned by tests/golden).
"""
from __future__ import annotations

import ctypes as C
from collections import deque

from . import _lib
from .sequence import Sequence


class BlockManager:
    def __init__(self, num_blocks: int, block_size: int):
        if num_blocks <= 0:
            raise ValueError("num_blocks must be positive")
        self._lib = _lib.load()
        self._h = C.c_void_p()
        _lib.check(self._lib.infer_block_manager_create(C.byref(self._h), num_blocks, block_size), "BlockManager")
        self.num_blocks, self.block_size = num_blocks, block_size

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            self._lib.infer_block_manager_destroy(h)
            self._h = None

    def _fail(self, rc: int, what: str):
        if rc < 0:
            detail = self._lib.infer_block_manager_last_error(self._h).decode()
            raise RuntimeError(f"BlockManager.{what}: {self._lib.infer_strerror(int(rc)).decode()} ({detail})")
        return rc

    def _pull_table(self, seq: Sequence):
        n = self._fail(self._lib.infer_block_manager_block_table(self._h, seq.seq_id, None, 0), "block_table")
        buf = (C.c_int32 * max(n, 1))()
        self._lib.infer_block_manager_block_table(self._h, seq.seq_id, buf, n)
        seq.block_table[:] = list(buf[:n])

    # -- the scheduler's calls ---------------------------------------------------------------
    def can_allocate(self, seq: Sequence) -> bool:
        return self._fail(self._lib.infer_block_manager_can_allocate(self._h, len(seq)), "can_allocate") == 1

    def allocate(self, seq: Sequence):
        if seq.block_table:
            raise RuntimeError("sequence already has pages")
        ids = (C.c_int64 * len(seq))(*seq.token_ids)
        seq.num_cached_tokens = self._fail(self._lib.infer_block_manager_allocate(self._h, seq.seq_id, ids, len(seq)),
                                           "allocate")
        self._pull_table(seq)

    def deallocate(self, seq: Sequence):
        self._fail(self._lib.infer_block_manager_deallocate(self._h, seq.seq_id), "deallocate")
        seq.num_cached_tokens = 0
        seq.block_table.clear()

    def can_append(self, seq: Sequence) -> bool:
        # the reference asks with the token already appended on the Python side
        # (infer/engine/block_mannager.py:114-115): one page is needed when it starts a new one
        return self.num_free() >= (1 if len(seq) % self.block_size == 1 else 0)

    def may_append(self, seq: Sequence):
        """Called after ``seq.append_token``: hands the tokens the allocator has not seen yet to the
        native side, which opens a page or seals one as the reference does
        (infer/engine/block_mannager.py:117-133)."""
        known = self._fail(self._lib.infer_block_manager_num_tokens(self._h, seq.seq_id), "may_append")
        new = seq.token_ids[known:]
        ids = (C.c_int64 * max(len(new), 1))(*new)
        self._fail(self._lib.infer_block_manager_append(self._h, seq.seq_id, ids, len(new)), "may_append")
        if len(seq.block_table) != -(-len(seq) // self.block_size):
            self._pull_table(seq)

    # -- accounting ----------------------------------------------------------------------------
    def num_free(self) -> int:
        return self._lib.infer_block_manager_num_free(self._h)

    def ref_counts(self) -> list[int]:
        buf = (C.c_int32 * self.num_blocks)()
        self._lib.infer_block_manager_ref_counts(self._h, buf, self.num_blocks)
        return list(buf)

    @property
    def free_block_ids(self) -> deque:
        n = self.num_free()
        buf = (C.c_int32 * max(n, 1))()
        self._lib.infer_block_manager_free_ids(self._h, buf, n)
        return deque(buf[:n])

    @free_block_ids.setter
    def free_block_ids(self, order):
        """Re-orders the free list (every page free): workload generators scatter pages with it."""
        order = list(order)
        buf = (C.c_int32 * max(len(order), 1))(*order)
        self._fail(self._lib.infer_block_manager_set_free_order(self._h, buf, len(order)), "free_block_ids")
