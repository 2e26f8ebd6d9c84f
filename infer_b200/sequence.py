"""``Sequence``: what the host side knows about one request.

It carries the attributes the step-metadata builders read off a request - the token ids, the
logical -> physical page list the allocator fills in, and the number of prompt tokens whose
pages were found in the prefix cache - under the names the reference's runner uses
(infer/engine/model_runner.py:66-126 reads ``len(seq)``, ``seq.block_table``,
``seq.num_cached_tokens``, ``seq.num_cached_blocks``, ``seq.num_blocks``,
``seq.last_block_num_tokens``, ``seq.last_token``; infer/engine/sequence.py:15-84 defines them).
Page allocation itself is native code (``BlockManager``).
"""
from __future__ import annotations

import itertools

_next_id = itertools.count()


class Sequence:
    block_size = 256          # page size in tokens (the engine config requires a multiple of 256)

    def __init__(self, token_ids, max_tokens: int = 64):
        self.seq_id = next(_next_id)
        self.token_ids = [int(t) for t in token_ids]
        if not self.token_ids:
            raise ValueError("a sequence needs at least one token")
        self.num_prompt_tokens = len(self.token_ids)
        self.max_tokens = max_tokens
        self.num_cached_tokens = 0
        self.block_table: list[int] = []

    def __len__(self):
        return len(self.token_ids)

    def __getitem__(self, key):
        return self.token_ids[key]

    @property
    def last_token(self) -> int:
        return self.token_ids[-1]

    @property
    def num_completion_tokens(self) -> int:
        return len(self.token_ids) - self.num_prompt_tokens

    @property
    def num_blocks(self) -> int:
        return -(-len(self.token_ids) // self.block_size)

    @property
    def num_cached_blocks(self) -> int:
        return self.num_cached_tokens // self.block_size

    @property
    def last_block_num_tokens(self) -> int:
        return len(self.token_ids) - (self.num_blocks - 1) * self.block_size

    def append_token(self, token_id: int):
        self.token_ids.append(int(token_id))
