"""``Attention`` module with the reference's constructor and forward contract
(infer/ops/attention.py:47-122): append the new k/v rows to the layer's page pools, then
run paged prefill or paged decode attention according to the step's ``Context``."""
from __future__ import annotations

import torch

from . import ops
from .context import get_context


class Attention(torch.nn.Module):
    def __init__(self, num_heads: int, head_dim: int, scale: float, num_kv_heads: int):
        super().__init__()
        self.num_heads, self.head_dim, self.scale, self.num_kv_heads = num_heads, head_dim, scale, num_kv_heads
        self.k_cache = self.v_cache = torch.tensor([])
        self.k_scale = self.v_scale = None        # set together with uint8 pools for FP8 KV

    def forward(self, Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor) -> torch.Tensor:
        Q = Q.view(-1, self.num_heads, self.head_dim)
        K = K.view(-1, self.num_kv_heads, self.head_dim)
        V = V.view(-1, self.num_kv_heads, self.head_dim)
        ctx = get_context()
        if not (self.k_cache.numel() and self.v_cache.numel()):
            raise RuntimeError("Attention: the layer has no page pools (allocate_kv_cache not run)")
        if not ctx.is_prefill and self.k_scale is None:
            # bf16 decode step: append and attention in one launch.  The slot of a sequence's new token follows from
            # context_lens and block_tables (position context_len - 1), which is what prepare_decode's slot_mapping
            # holds as well (infer/engine/model_runner.py:110-126); rows with context_len 0 (the padding of a
            # captured batch, slot -1 there) are skipped by both.
            O = ops.paged_attn_decode_append(Q.contiguous(), K, V, self.k_cache, self.v_cache, ctx.context_lens,
                                             ctx.block_tables, self.scale)
            return O.view(-1, self.num_heads * self.head_dim)
        ops.store_kvcache(K, V, self.k_cache, self.v_cache, ctx.slot_mapping, self.k_scale, self.v_scale)
        if ctx.is_prefill:
            block_tables = ctx.block_tables
            if block_tables is None:
                raise RuntimeError("Attention: prefill needs block_tables (keys are read from the pools)")
            O = ops.paged_attn_prefill(Q.contiguous(), self.k_cache, self.v_cache, ctx.cu_seqlens_q, ctx.cu_seqlens_k,
                                       ctx.max_seqlen_q, ctx.max_seqlen_k, self.scale, block_tables)
        else:
            O = ops.paged_attn_decode(Q.contiguous(), self.k_cache, self.v_cache, ctx.context_lens, ctx.block_tables,
                                      self.scale, k_scale=self.k_scale, v_scale=self.v_scale)
        return O.view(-1, self.num_heads * self.head_dim)
