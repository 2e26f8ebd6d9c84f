"""Per-request token list and its page table.

Host-side mirror of the reference's ``Sequence`` (infer/engine/sequence.py:15-84):
same attribute names and the same page arithmetic, so that the page allocator and
the step-metadata builders of this package read like the reference's callers.
Only what the paged KV path needs is kept (no sampling state machine).
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass
from enum import Enum, auto


@dataclass
class SamplingParams:
    """Mirror of infer/sampling_params.py (fields used by ``Sequence``)."""
    temperature: float = 1.0
    max_tokens: int = 64
    ignore_eos: bool = False


class SequenceStatus(Enum):
    WAITING = auto()
    RUNNING = auto()
    FINISHED = auto()


class Sequence:
    """A request: token ids plus the logical->physical page list.

    ``block_size`` is the page size in tokens (reference: 256,
    infer/engine/sequence.py:16; the engine config requires a multiple of 256,
    infer/config.py:21).
    """

    block_size = 256
    _ids = itertools.count()

    def __init__(self, token_ids, sampling_param: SamplingParams | None = None):
        sampling_param = sampling_param or SamplingParams()
        self.seq_id = next(Sequence._ids)
        self.status = SequenceStatus.WAITING
        self.token_ids = list(token_ids)
        self.num_tokens = len(self.token_ids)
        self.num_prompt_tokens = self.num_tokens
        self.last_token = self.token_ids[-1]
        self.num_cached_tokens = 0
        self.block_table: list[int] = []
        self.temperature = sampling_param.temperature
        self.max_tokens = sampling_param.max_tokens
        self.ignore_eos = sampling_param.ignore_eos

    def __len__(self):
        return self.num_tokens

    def __getitem__(self, key):
        return self.token_ids[key]

    @property
    def num_cached_blocks(self) -> int:
        return self.num_cached_tokens // self.block_size

    @property
    def num_blocks(self) -> int:
        return -(-self.num_tokens // self.block_size)

    @property
    def last_block_num_tokens(self) -> int:
        return self.num_tokens - (self.num_blocks - 1) * self.block_size

    def block(self, i: int):
        """Token ids held by logical page ``i``."""
        if not 0 <= i < self.num_blocks:
            raise IndexError(i)
        lo = i * self.block_size
        return self.token_ids[lo:lo + self.block_size]

    def append_token(self, token_id: int):
        self.token_ids.append(token_id)
        self.last_token = token_id
        self.num_tokens += 1
