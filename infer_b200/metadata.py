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
