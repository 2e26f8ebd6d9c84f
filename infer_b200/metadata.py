"""Step metadata: slot_mapping, block_tables, context_lens, cu_seqlens.

These are the integer tensors the reference's ``ModelRunner`` builds before every
forward pass (infer/engine/model_runner.py:66-126) and that define the input
layout of the append and attention kernels:

* ``block_tables``  int32 [B, max_pages], ragged rows padded with -1;
* decode: ``context_lens`` int32 [B] counts the token being appended, and that
  token's slot is ``block_table[-1] * block_size + last_block_num_tokens - 1``;
* prefill: ``cu_seqlens_q`` runs over the new (uncached) tokens, ``cu_seqlens_k``
  over whole sequences; ``slot_mapping`` lists every slot of the pages that are not
  prefix-cache hits; ``block_tables`` is only built when some prefix is cached.

``prepare_chunk`` generalises the prefill rule to a chunk that starts at any token
position (the reference only ever starts on a page boundary, because its prefix
cache works in whole pages).
"""
from __future__ import annotations

import torch

from .context import set_context
from .sequence import Sequence


def _to(t: torch.Tensor, device):
    if device is None or torch.device(device).type == "cpu":
        return t
    return t.pin_memory().to(device, non_blocking=True)


def prepare_block_tables(seqs: list[Sequence], device=None, width: int | None = None) -> torch.Tensor:
    """infer/engine/model_runner.py:66-70."""
    width = max(len(s.block_table) for s in seqs) if width is None else width
    rows = [s.block_table + [-1] * (width - len(s.block_table)) for s in seqs]
    return _to(torch.tensor(rows, dtype=torch.int32), device)


def prepare_decode(seqs: list[Sequence], block_size: int, device=None):
    """infer/engine/model_runner.py:110-126.  Returns (input_ids, positions) and
    publishes slot_mapping / context_lens / block_tables through the Context."""
    input_ids, positions, slots, lens = [], [], [], []
    for s in seqs:
        input_ids.append(s.last_token)
        positions.append(len(s))
        lens.append(len(s))
        slots.append(s.block_table[-1] * block_size + s.last_block_num_tokens - 1)
    slot_mapping = _to(torch.tensor(slots, dtype=torch.int32), device)
    context_lens = _to(torch.tensor(lens, dtype=torch.int32), device)
    block_tables = prepare_block_tables(seqs, device)
    set_context(False, slot_mapping=slot_mapping, context_lens=context_lens, block_tables=block_tables)
    return (_to(torch.tensor(input_ids, dtype=torch.int64), device),
            _to(torch.tensor(positions, dtype=torch.int64), device))


def prepare_prefill(seqs: list[Sequence], block_size: int, device=None):
    """infer/engine/model_runner.py:72-108."""
    input_ids, positions, slots = [], [], []
    cu_q, cu_k = [0], [0]
    max_q = max_k = 0
    for s in seqs:
        n = len(s)
        input_ids.extend(s[s.num_cached_tokens:])
        positions.extend(range(s.num_cached_tokens, n))
        nq = n - s.num_cached_tokens
        cu_q.append(cu_q[-1] + nq)
        cu_k.append(cu_k[-1] + n)
        max_q, max_k = max(max_q, nq), max(max_k, n)
        if not s.block_table:
            continue
        for i in range(s.num_cached_blocks, s.num_blocks):
            lo = s.block_table[i] * block_size
            fill = block_size if i != s.num_blocks - 1 else s.last_block_num_tokens
            slots.extend(range(lo, lo + fill))
    block_tables = prepare_block_tables(seqs, device) if cu_k[-1] > cu_q[-1] else None
    set_context(True,
                _to(torch.tensor(cu_q, dtype=torch.int32), device),
                _to(torch.tensor(cu_k, dtype=torch.int32), device),
                max_q, max_k,
                _to(torch.tensor(slots, dtype=torch.int32), device),
                None, block_tables)
    return (_to(torch.tensor(input_ids, dtype=torch.int64), device),
            _to(torch.tensor(positions, dtype=torch.int64), device))


def chunk_slots(block_table: list[int], start: int, stop: int, block_size: int) -> list[int]:
    """Slots of token positions [start, stop) of one sequence:
    ``block_table[pos // block_size] * block_size + pos % block_size``."""
    return [block_table[p // block_size] * block_size + p % block_size for p in range(start, stop)]


def prepare_chunk(block_tables: list[list[int]], prefix_lens: list[int], chunk_lens: list[int],
                  block_size: int, device=None):
    """Chunked prefill over cached prefixes of arbitrary length: queries are the
    chunk tokens, keys are prefix + chunk; always publishes block_tables."""
    cu_q, cu_k, slots = [0], [0], []
    for bt, p, c in zip(block_tables, prefix_lens, chunk_lens):
        cu_q.append(cu_q[-1] + c)
        cu_k.append(cu_k[-1] + p + c)
        slots.extend(chunk_slots(bt, p, p + c, block_size))
    width = max(len(bt) for bt in block_tables)
    rows = [bt + [-1] * (width - len(bt)) for bt in block_tables]
    set_context(True,
                _to(torch.tensor(cu_q, dtype=torch.int32), device),
                _to(torch.tensor(cu_k, dtype=torch.int32), device),
                max(chunk_lens), max(p + c for p, c in zip(prefix_lens, chunk_lens)),
                _to(torch.tensor(slots, dtype=torch.int32), device),
                None, _to(torch.tensor(rows, dtype=torch.int32), device))


class DecodeState:
    """Decode-step metadata kept on the device between steps.

    ``prepare_decode`` rebuilds and uploads everything every step; this class uploads once and
    then lets ``advance()`` (one small kernel) grow every live sequence by one token and compute
    the new slots and positions from the block tables already on the device.  The host only
    writes a block-table entry when a sequence enters a new page.  All tensors keep their
    address, so they can be the static inputs of a captured decode graph
    (infer/engine/model_runner.py:163-198 uses the same static-buffer scheme)."""

    def __init__(self, max_batch: int, max_pages: int, block_size: int, device, position_base: int = 1):
        self.block_size, self.position_base, self.device = block_size, position_base, torch.device(device)
        self.context_lens = torch.zeros(max_batch, dtype=torch.int32, device=device)
        self.slot_mapping = torch.full((max_batch,), -1, dtype=torch.int32, device=device)
        self.positions = torch.zeros(max_batch, dtype=torch.int64, device=device)
        self.block_tables = torch.full((max_batch, max_pages), -1, dtype=torch.int32, device=device)
        self.host_lens = [0] * max_batch
        self.host_pages = [0] * max_batch          # pages known to the device per row

    def load(self, seqs: list[Sequence], pending: int = 0):
        """Full upload for a new batch composition; lengths are those BEFORE the next step's token.
        ``pending``: tokens at the end of every sequence that the coming ``advance()`` calls will count (1 when the
        engine has already appended the sampled token whose k/v the next step stores)."""
        n, width = len(seqs), self.block_tables.shape[1]
        if n > self.context_lens.numel() or any(len(s.block_table) > width for s in seqs):
            raise ValueError("batch or page list exceeds the static buffers")
        lens = [len(s) - pending for s in seqs] + [0] * (self.context_lens.numel() - n)
        rows = [s.block_table + [-1] * (width - len(s.block_table)) for s in seqs]
        rows += [[-1] * width] * (self.context_lens.numel() - n)
        self.context_lens.copy_(torch.tensor(lens, dtype=torch.int32), non_blocking=True)
        self.block_tables.copy_(torch.tensor(rows, dtype=torch.int32), non_blocking=True)
        self.host_lens = lens
        self.host_pages = [len(s.block_table) for s in seqs] + [0] * (self.context_lens.numel() - n)

    def publish_new_pages(self, seqs: list[Sequence]):
        """After the allocator ran ``may_append`` for the coming step: upload only the
        block-table entries that did not exist yet."""
        for b, s in enumerate(seqs):
            have = self.host_pages[b]
            if len(s.block_table) > have:
                new = torch.tensor(s.block_table[have:], dtype=torch.int32)
                self.block_tables[b, have:len(s.block_table)].copy_(new, non_blocking=True)
                self.host_pages[b] = len(s.block_table)

    def advance(self):
        """One kernel: context_lens += 1 for live rows, slot_mapping and positions follow."""
        if self.device.type != "cuda":
            raise RuntimeError("DecodeState.advance launches a CUDA kernel; the state must live on a GPU")
        import ctypes as C
        from . import _lib
        lib = _lib.load()
        p = lambda t: C.c_void_p(t.data_ptr())
        with torch.cuda.device(self.device):
            rc = lib.infer_decode_step_advance(p(self.context_lens), p(self.slot_mapping), p(self.positions),
                                               p(self.block_tables), self.block_tables.stride(0),
                                               self.context_lens.numel(), self.block_size, self.position_base,
                                               C.c_void_p(torch.cuda.current_stream().cuda_stream))
        _lib.check(rc, "decode_step_advance")
        self.host_lens = [n + 1 if n > 0 else 0 for n in self.host_lens]
        set_context(False, slot_mapping=self.slot_mapping, context_lens=self.context_lens,
                    block_tables=self.block_tables)
