"""CPU oracle for the paged KV-cache path.  TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may import
this module; nothing in ``infer_b200`` does, and the CUDA path never falls back to it.

What it restates (reference paths are relative to the Graylatzhou/Infer tree):

* ``store_kvcache``      infer/ops/attention.py:16-45  - row ``i`` of key/value goes to
                         flat slot ``slot_mapping[i]`` of the pool, all ``Hkv*d`` elements.
* ``paged_decode``       infer/ops/attention.py:117-121 - what the reference obtains from
                         ``flash_attn_with_kvcache(q[:,None], k_cache, v_cache,
                         cache_seqlens, block_table, softmax_scale, causal=True)``.
* ``paged_prefill``      infer/ops/attention.py:110-116 - ``flash_attn_varlen_func`` with a
                         block table: keys are prefix + chunk, causal mask aligned to the
                         bottom-right corner (chunk token i sees prefix + i + 1 keys).
* ``dense_causal``       src/operators/flashattn/flashattn.cu:40-328 as pinned by
                         test/op.py:269-287: Q,K,V,O [B,H,S,128], SDPA is_causal=True,
                         GQA by kv_head = head // (Hq/Hkv) (flashattn.cu:76).
* pool geometry          infer/engine/model_runner.py:55-64: [num_blocks, block_size, Hkv, d].

The attention arithmetic itself lives in the third-party ``flash_attn`` package
(imported at infer/ops/attention.py:3; no version is pinned by the reference, 2.8.3 is
the one in this image), which has no CPU path.  The oracle restates its published
algorithm - softmax(scale * q k^T) v over the first ``context_len`` tokens in fp32 -
and rounds once to the output dtype.

Pinning status: the append and all integer metadata are pinned bit-exactly by golden
vectors produced by the reference's own code (tests/golden/make_golden.py runs the
reference's Triton store kernel under the Triton interpreter, its BlockManager and its
ModelRunner.prepare_* on CPU).  The attention outputs are pinned against
``torch.nn.functional.scaled_dot_product_attention`` (the expected-value function of the
reference's own attention test, test/op.py:278-281) on the same golden inputs.  The FP8
KV format has no counterpart in the reference: for it this oracle is the definition
(parity unpinned).

FP8 rule (e4m3, one fp32 scale per (page, kv head)):
  scale  = amax(|x| over the rows of that page/head written so far) / 448   (fp32 division)
  stored = e4m3_rne(clamp(x / scale, -448, 448)); scale 0 (all-zero page) stores zeros.
  When an append raises a page's scale from old > 0 to new, every row of that page/head is
  first re-encoded as e4m3_rne(float(stored) * (old / new)), then the new rows are written.
"""
from __future__ import annotations

import math

import torch

E4M3_MAX = 448.0


# --------------------------------------------------------------------------- append
def store_kvcache(key, value, k_cache, v_cache, slot_mapping):
    """In-place scatter of [N, Hkv, d] rows into [num_blocks, block_size, Hkv, d] pools.
    Rows whose slot is negative are skipped (padding rows of a captured batch)."""
    n, hkv, d = key.shape
    assert slot_mapping.numel() == n
    keep = slot_mapping >= 0
    idx = slot_mapping[keep].long()
    k_cache.view(-1, hkv, d).index_copy_(0, idx, key[keep].to(k_cache.dtype))
    v_cache.view(-1, hkv, d).index_copy_(0, idx, value[keep].to(v_cache.dtype))


def _to_e4m3(x: torch.Tensor) -> torch.Tensor:
    return x.clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)


def store_kvcache_fp8(key, value, k_cache, v_cache, k_scale, v_scale, slot_mapping):
    """FP8 append.  Pools are uint8 views of e4m3 bytes [num_blocks, block_size, Hkv, d];
    scales are fp32 [num_blocks, Hkv].  See the module docstring for the rule."""
    n, hkv, d = key.shape
    block_size = k_cache.shape[1]
    keep = slot_mapping >= 0
    slots = slot_mapping[keep].long()
    pages = slots // block_size
    for x, cache, scale in ((key[keep], k_cache, k_scale), (value[keep], v_cache, v_scale)):
        xf = x.float()
        row_s = xf.abs().amax(dim=-1) / E4M3_MAX                       # [n, Hkv]
        bytes_ = cache.view(torch.float8_e4m3fn)
        for p in torch.unique(pages).tolist():
            cand = row_s[pages == p].amax(dim=0)                       # [Hkv]
            old = scale[p].clone()
            new = torch.maximum(old, cand)
            grew = (new > old) & (old > 0)
            for h in torch.nonzero(grew).flatten().tolist():
                ratio = old[h] / new[h]
                bytes_[p, :, h, :] = _to_e4m3(bytes_[p, :, h, :].float() * ratio)
            scale[p] = new
        s = scale[pages]                                               # [n, Hkv]
        q = torch.where(s[..., None] > 0, xf / s[..., None], torch.zeros_like(xf))
        bytes_.view(-1, hkv, d).view(torch.uint8).index_copy_(0, slots, _to_e4m3(q).view(torch.uint8))


# --------------------------------------------------------------------------- fused pre-attention step
def rms_norm_heads(x, weight, eps):
    """Per-head RMSNorm as the reference computes it (RMSNorm.rms_forward,
    infer/ops/norm.py:63-73): fp32 variance and scaling, round to the input dtype, then a
    multiply by the weight in that dtype."""
    dt = x.dtype
    xf = x.to(torch.float32)
    var = xf.pow(2).mean(dim=-1, keepdim=True)
    xf = xf * torch.rsqrt(var + eps)
    return xf.to(dt) * weight


def rope_neox(x, cos, sin):
    """GPT-NeoX rotary embedding in the tensor's own dtype, the arithmetic of
    _apply_rotary_emb_torch (infer/ops/rope.py:46-64) and of the CUDA op
    (src/operators/rope/rope.cu:43-66): x [T, H, d], cos/sin [T, d/2]."""
    cos = cos.unsqueeze(-2).to(x.dtype)
    sin = sin.unsqueeze(-2).to(x.dtype)
    x1, x2 = torch.chunk(x, 2, dim=-1)
    return torch.cat((x1 * cos - x2 * sin, x2 * cos + x1 * sin), dim=-1)


def qk_norm_rope_append(q, k, v, q_weight, k_weight, eps, positions, cos_sin_cache, k_cache, v_cache, slot_mapping):
    """What the reference model does between the qkv projection and attention
    (infer/models/Qwen3.py:112-131): norm q and k per head, rotate both in place, store k and v.
    Returns the rotated q; the pools are updated in place."""
    cos, sin = cos_sin_cache.index_select(0, positions).chunk(2, dim=-1)
    qn = rope_neox(rms_norm_heads(q, q_weight, eps), cos, sin)
    kn = rope_neox(rms_norm_heads(k, k_weight, eps), cos, sin)
    store_kvcache(kn, v, k_cache, v_cache, slot_mapping)
    return qn


# --------------------------------------------------------------------------- gather
def gather_tokens(cache, table_row, length, scale=None):
    """Rows [0, length) of one sequence, found by walking its page list.
    Returns fp32 [length, Hkv, d]; e4m3 pools are dequantised with their page scales."""
    block_size = cache.shape[1]
    n_pages = -(-length // block_size)
    pages = table_row[:n_pages].long()
    assert bool((pages >= 0).all()), "page list shorter than the context"
    if scale is None:
        rows = cache[pages].float()
    else:
        rows = cache[pages].view(torch.float8_e4m3fn).float() * scale[pages][:, None, :, None]
    return rows.reshape(n_pages * block_size, *cache.shape[2:])[:length]


# --------------------------------------------------------------------------- attention
def _attend(q, k, v, scale, mask=None):
    """q [Lq,Hq,d], k/v [Lk,Hkv,d] fp32 -> [Lq,Hq,d] fp32."""
    g = q.shape[1] // k.shape[1]
    k = k.repeat_interleave(g, dim=1)
    v = v.repeat_interleave(g, dim=1)
    s = torch.einsum("qhd,khd->hqk", q, k) * scale
    if mask is not None:
        s = s.masked_fill(~mask[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.einsum("hqk,khd->qhd", p, v)


def paged_decode(q, k_cache, v_cache, context_lens, block_tables, scale,
                 k_scale=None, v_scale=None, out_dtype=torch.bfloat16):
    """q [B,Hq,d] -> [B,Hq,d].  Rows with context_len == 0 stay zero."""
    out = torch.zeros(q.shape, dtype=torch.float32)
    for b in range(q.shape[0]):
        length = int(context_lens[b])
        if length == 0:
            continue
        k = gather_tokens(k_cache, block_tables[b], length, k_scale)
        v = gather_tokens(v_cache, block_tables[b], length, v_scale)
        out[b] = _attend(q[b:b + 1].float(), k, v, scale)[0]
    return out.to(out_dtype)


def paged_prefill(q, k_cache, v_cache, cu_seqlens_q, cu_seqlens_k, block_tables, scale,
                  out_dtype=torch.bfloat16, q_block=1024):
    """q [sum_q,Hq,d] -> [sum_q,Hq,d]; keys of sequence b are its first
    cu_k[b+1]-cu_k[b] cached tokens (the chunk must already be appended)."""
    out = torch.zeros(q.shape, dtype=torch.float32)
    for b in range(cu_seqlens_q.numel() - 1):
        q0, q1 = int(cu_seqlens_q[b]), int(cu_seqlens_q[b + 1])
        lk = int(cu_seqlens_k[b + 1]) - int(cu_seqlens_k[b])
        lq = q1 - q0
        if lq == 0:
            continue
        k = gather_tokens(k_cache, block_tables[b], lk)
        v = gather_tokens(v_cache, block_tables[b], lk)
        kpos = torch.arange(lk)
        for s in range(0, lq, q_block):
            e = min(lq, s + q_block)
            qpos = torch.arange(s, e) + (lk - lq)
            mask = kpos[None, :] <= qpos[:, None]
            out[q0 + s:q0 + e] = _attend(q[q0 + s:q0 + e].float(), k, v, scale, mask)
    return out.to(out_dtype)


def dense_causal(Q, K, V, out_dtype=torch.bfloat16):
    """Q [B,Hq,S,d], K/V [B,Hkv,S,d] -> O [B,Hq,S,d]; scale 1/sqrt(d) as the reference op
    computes it internally (flashattn.cu:293)."""
    b, hq, s, d = Q.shape
    scale = 1.0 / math.sqrt(d)
    mask = torch.ones(s, s, dtype=torch.bool).tril()
    out = torch.empty(Q.shape, dtype=torch.float32)
    for i in range(b):
        o = _attend(Q[i].float().transpose(0, 1), K[i].float().transpose(0, 1),
                    V[i].float().transpose(0, 1), scale, mask)
        out[i] = o.transpose(0, 1)
    return out.to(out_dtype)


# --------------------------------------------------------------------------- timed flavour
def paged_decode_bf16_sdpa(q, k_cache, v_cache, context_lens, block_tables, scale):
    """The same decode step the way the reference's torch path would run it on CPU:
    page gather + ``F.scaled_dot_product_attention`` in bf16 (Attention.forward_native,
    infer/ops/attention.py:64-71).  Used as the timed CPU baseline, not as the checker."""
    block_size = k_cache.shape[1]
    g = q.shape[1] // k_cache.shape[2]
    out = torch.zeros_like(q)
    for b in range(q.shape[0]):
        length = int(context_lens[b])
        if length == 0:
            continue
        pages = block_tables[b, :-(-length // block_size)].long()
        k = k_cache[pages].reshape(-1, *k_cache.shape[2:])[:length]
        v = v_cache[pages].reshape(-1, *v_cache.shape[2:])[:length]
        k = k.transpose(0, 1).repeat_interleave(g, dim=0)          # [Hq, L, d]
        v = v.transpose(0, 1).repeat_interleave(g, dim=0)
        o = torch.nn.functional.scaled_dot_product_attention(
            q[b][:, None, :], k, v, scale=scale)                     # [Hq, 1, d]
        out[b] = o[:, 0, :]
    return out
