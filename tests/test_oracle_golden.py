"""The CPU oracle and the host-side mirrors against golden vectors produced by the
reference's own code (tests/golden/make_golden.py)."""
import hashlib
from pathlib import Path

import numpy as np
import torch

from infer_b200 import BlockManager, Sequence, get_context
from infer_b200 import metadata
from oracle import paged_kv_oracle as oracle

GOLD = Path(__file__).resolve().parent / "golden"


def digest(t):
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def test_append_matches_reference_store_kernel(golden):
    g = golden["append"]
    gen = torch.Generator().manual_seed(g["seed"])
    n, hq, hkv, d = g["n"], g["hq"], g["hkv"], 128
    qkv = torch.randn(n, (hq + 2 * hkv) * d, generator=gen).bfloat16()
    assert digest(qkv) == g["qkv_digest"], "seeded inputs differ from the ones the fixture was made with"
    key = qkv[:, hq * d:(hq + hkv) * d].view(n, hkv, d)
    value = qkv[:, (hq + hkv) * d:].view(n, hkv, d)
    k_cache = torch.zeros(g["num_blocks"], 256, hkv, d, dtype=torch.bfloat16)
    v_cache = torch.zeros_like(k_cache)
    oracle.store_kvcache(key, value, k_cache, v_cache, torch.tensor(g["slots"], dtype=torch.int32))
    assert digest(k_cache) == g["k_cache_digest"]
    assert digest(v_cache) == g["v_cache_digest"]


def test_append_skips_negative_slots():
    k = torch.randn(3, 2, 128, generator=torch.Generator().manual_seed(3)).bfloat16()
    kc = torch.zeros(1, 256, 2, 128, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    oracle.store_kvcache(k, k, kc, vc, torch.tensor([5, -1, 7], dtype=torch.int32))
    assert torch.equal(kc[0, 5], k[0]) and torch.equal(kc[0, 7], k[2])
    untouched = torch.ones(256, dtype=torch.bool)
    untouched[[5, 7]] = False
    assert not kc[0, untouched].any() and not vc[0, untouched].any()      # the skipped row went nowhere


def _replay(golden):
    g = golden["allocator"]
    mgr = BlockManager(g["num_blocks"], g["block_size"])
    seqs = []
    for p in g["prompts"]:
        s = Sequence(p)
        mgr.allocate(s)
        seqs.append(s)
    yield "prefill", mgr, seqs
    for step, toks in enumerate(g["new_tokens"]):
        for s, t in zip(seqs, toks):
            s.append_token(t)
            mgr.may_append(s)
        yield f"decode{step}", mgr, seqs
    mgr.deallocate(seqs[0])
    mgr.deallocate(seqs[2])
    yield "freed", mgr, seqs
    late = Sequence(g["late_prompt"])
    mgr.allocate(late)
    seqs.append(late)
    yield "late_prefill", mgr, seqs


def test_block_manager_matches_reference(golden):
    events = {e["tag"]: e for e in golden["allocator"]["events"]}
    seen = 0
    for tag, mgr, seqs in _replay(golden):
        e = events[tag]
        assert [list(s.block_table) for s in seqs] == e["tables"], tag
        assert [s.num_cached_tokens for s in seqs] == e["cached"], tag
        assert mgr.ref_counts() == e["ref_counts"], tag
        assert list(mgr.free_block_ids) == e["free"], tag
        seen += 1
    assert seen == len(events)


def _check_context(e):
    c = get_context()
    ref = e["context"]
    for name in ("cu_seqlens_q", "cu_seqlens_k", "slot_mapping", "context_lens", "block_tables"):
        mine = getattr(c, name)
        assert (None if mine is None else mine.tolist()) == ref[name], name
        if mine is not None:
            assert mine.dtype == torch.int32
    assert c.max_seqlen_q == ref["max_seqlen_q"] and c.max_seqlen_k == ref["max_seqlen_k"]
    assert c.is_prefill == ref["is_prefill"]


def test_step_metadata_matches_reference(golden):
    events = {e["tag"]: e for e in golden["allocator"]["events"]}
    bs = golden["allocator"]["block_size"]
    for tag, mgr, seqs in _replay(golden):
        if tag == "prefill":
            metadata.prepare_prefill(seqs, bs)
            _check_context(events[tag])
        elif tag.startswith("decode"):
            metadata.prepare_decode(seqs, bs)
            _check_context(events[tag])
        elif tag == "late_prefill":
            metadata.prepare_prefill([seqs[-1]], bs)
            _check_context(events[tag])


def test_dense_causal_matches_sdpa(golden):
    g = golden["attention"]
    gen = torch.Generator().manual_seed(g["seed"])
    Q = torch.randn(1, 4, 64, 128, generator=gen).bfloat16()
    K = torch.randn(1, 4, 64, 128, generator=gen).bfloat16()
    V = torch.randn(1, 4, 64, 128, generator=gen).bfloat16()
    assert digest(torch.cat([Q, K, V])) == g["dense_inputs_digest"]
    want = torch.from_numpy(np.load(GOLD / "dense_causal_O.npy")).view(torch.bfloat16)
    got = oracle.dense_causal(Q, K, V)
    # the reference's own tolerance for this op (test/op.py:283)
    torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=1e-3)


def test_paged_decode_matches_sdpa_on_paged_copy(golden):
    """Lay the golden keys out in scattered pages; the oracle's paged decode must give what
    SDPA gave on the contiguous keys."""
    g = golden["attention"]
    gen = torch.Generator().manual_seed(g["seed"])
    for _ in range(3):
        torch.randn(1, 4, 64, 128, generator=gen)          # skip the dense tensors
    lens, hq, hkv = g["decode_lens"], g["decode_hq"], g["decode_hkv"]
    want = torch.from_numpy(np.load(GOLD / "decode_sdpa_O.npy"))
    num_blocks = 16
    k_cache = torch.randn(num_blocks, 256, hkv, 128).bfloat16()   # stale content everywhere
    v_cache = torch.randn(num_blocks, 256, hkv, 128).bfloat16()
    perm = torch.randperm(num_blocks, generator=torch.Generator().manual_seed(1)).tolist()
    tables, qs, at = [], [], 0
    dig = hashlib.sha256()
    for n in lens:
        q = torch.randn(hq, 1, 128, generator=gen).bfloat16()
        k = torch.randn(hkv, n, 128, generator=gen).bfloat16()
        v = torch.randn(hkv, n, 128, generator=gen).bfloat16()
        dig.update(digest(torch.cat([q.flatten(), k.flatten(), v.flatten()])).encode())
        pages = perm[at:at + -(-n // 256)]
        at += len(pages)
        slots = torch.tensor(metadata.chunk_slots(pages, 0, n, 256), dtype=torch.int32)
        oracle.store_kvcache(k.transpose(0, 1).contiguous(), v.transpose(0, 1).contiguous(), k_cache, v_cache, slots)
        tables.append(pages + [-1] * (3 - len(pages)))
        qs.append(q[:, 0, :])
    assert dig.hexdigest() == g["decode_inputs_digest"]
    got = oracle.paged_decode(torch.stack(qs), k_cache, v_cache, torch.tensor(lens, dtype=torch.int32),
                              torch.tensor(tables, dtype=torch.int32), 128 ** -0.5, out_dtype=torch.float32)
    torch.testing.assert_close(got, want, atol=1e-5, rtol=1e-5)
    got_bf16 = oracle.paged_decode_bf16_sdpa(torch.stack(qs), k_cache, v_cache, torch.tensor(lens, dtype=torch.int32),
                                             torch.tensor(tables, dtype=torch.int32), 128 ** -0.5)
    torch.testing.assert_close(got_bf16.float(), want, atol=2e-2, rtol=1e-2)


def test_prefill_equals_dense_causal_when_no_prefix():
    gen = torch.Generator().manual_seed(3)
    s, hq, hkv = 300, 4, 2
    q = torch.randn(s, hq, 128, generator=gen).bfloat16()
    k = torch.randn(s, hkv, 128, generator=gen).bfloat16()
    v = torch.randn(s, hkv, 128, generator=gen).bfloat16()
    kc = torch.zeros(4, 256, hkv, 128, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    pages = [2, 0]
    oracle.store_kvcache(k, v, kc, vc, torch.tensor(metadata.chunk_slots(pages, 0, s, 256), dtype=torch.int32))
    cu = torch.tensor([0, s], dtype=torch.int32)
    got = oracle.paged_prefill(q, kc, vc, cu, cu, torch.tensor([pages], dtype=torch.int32), 128 ** -0.5)
    want = oracle.dense_causal(q.transpose(0, 1)[None], k.transpose(0, 1)[None], v.transpose(0, 1)[None])[0].transpose(0, 1)
    torch.testing.assert_close(got.float(), want.float(), atol=1e-2, rtol=1e-2)


def test_prefill_last_row_equals_decode():
    """Bottom-right alignment: the last chunk row sees every key, like a decode step."""
    gen = torch.Generator().manual_seed(4)
    prefix, chunk, hq, hkv = 300, 70, 4, 2
    n = prefix + chunk
    kc = torch.randn(3, 256, hkv, 128, generator=gen).bfloat16()
    vc = torch.randn(3, 256, hkv, 128, generator=gen).bfloat16()
    q = torch.randn(chunk, hq, 128, generator=gen).bfloat16()
    table = torch.tensor([[1, 2, 0]], dtype=torch.int32)
    pre = oracle.paged_prefill(q, kc, vc, torch.tensor([0, chunk], dtype=torch.int32),
                               torch.tensor([0, n], dtype=torch.int32), table, 0.1)
    dec = oracle.paged_decode(q[-1:], kc, vc, torch.tensor([n], dtype=torch.int32), table, 0.1)
    assert torch.equal(pre[-1], dec[0])


def test_fp8_append_rule():
    gen = torch.Generator().manual_seed(5)
    hkv = 2
    kc = torch.zeros(2, 256, hkv, 128, dtype=torch.uint8)
    vc = torch.zeros_like(kc)
    ks = torch.zeros(2, hkv)
    vs = torch.zeros(2, hkv)
    k1 = torch.randn(10, hkv, 128, generator=gen).bfloat16()
    slots1 = torch.arange(10, dtype=torch.int32)
    oracle.store_kvcache_fp8(k1, k1, kc, vc, ks, vs, slots1)
    assert torch.allclose(ks[0], k1.float().abs().amax(dim=(0, 2)) / 448)
    assert ks[1].abs().sum() == 0
    deq = kc[0, :10].view(torch.float8_e4m3fn).float() * ks[0][None, :, None]
    assert (deq - k1.float()).abs().max() <= k1.float().abs().max() / 448 * 16 + 1e-6   # half an e4m3 ulp at the top binade
    before = kc.clone()
    # a louder row raises the scale: old rows are re-encoded, not left stale
    k2 = (torch.randn(1, hkv, 128, generator=gen) * 30).bfloat16()
    oracle.store_kvcache_fp8(k2, k2, kc, vc, ks, vs, torch.tensor([10], dtype=torch.int32))
    assert (ks[0] >= k2.float().abs().amax(dim=(0, 2)) / 448 - 1e-9).all()
    assert not torch.equal(before[0, :10], kc[0, :10])
    deq2 = kc[0, :10].view(torch.float8_e4m3fn).float() * ks[0][None, :, None]
    assert (deq2 - k1.float()).abs().max() <= ks[0].max() * 32 + 1e-6
    # a quieter row leaves scale and old rows alone
    before, s_before = kc.clone(), ks.clone()
    k3 = (torch.randn(1, hkv, 128, generator=gen) * 0.1).bfloat16()
    oracle.store_kvcache_fp8(k3, k3, kc, vc, ks, vs, torch.tensor([11], dtype=torch.int32))
    assert torch.equal(s_before, ks) and torch.equal(before[0, :11], kc[0, :11])


def _norm_rope_inputs(g):
    gen = torch.Generator().manual_seed(g["seed"])
    t, h, d = g["t"], g["h"], 128
    x = (torch.randn(t, h, d, generator=gen) * 1.7).bfloat16()
    weight = (1.0 + 0.1 * torch.randn(d, generator=gen)).bfloat16()
    inv_freq = 1.0 / (g["theta"] ** (torch.arange(0, d, 2, dtype=torch.bfloat16) / d))
    freqs = torch.einsum("i,j -> ij", torch.arange(g["max_position"], dtype=torch.bfloat16), inv_freq)
    cache = torch.cat((freqs.cos(), freqs.sin()), dim=-1)
    assert digest(torch.cat([x.flatten(), weight])) == g["inputs_digest"]
    assert digest(cache) == g["cache_digest"]
    return x, weight, cache, torch.tensor(g["positions"], dtype=torch.int64)


def test_norm_and_rope_match_reference_functions(golden):
    """rms_norm_heads and rope_neox against what the reference's RMSNorm.rms_forward and
    _apply_rotary_emb_torch produced on the same bits: bit-exact."""
    g = golden["norm_rope"]
    x, weight, cache, positions = _norm_rope_inputs(g)
    want_norm = torch.from_numpy(np.load(GOLD / "norm_only_out.npy")).view(torch.bfloat16)
    want = torch.from_numpy(np.load(GOLD / "norm_rope_out.npy")).view(torch.bfloat16)
    xn = oracle.rms_norm_heads(x, weight, g["eps"])
    assert torch.equal(xn.view(torch.int16), want_norm.view(torch.int16))
    cos, sin = cache.index_select(0, positions).chunk(2, dim=-1)
    got = oracle.rope_neox(xn, cos, sin)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))


def test_fused_oracle_equals_separate_steps(golden):
    g = golden["norm_rope"]
    x, weight, cache, positions = _norm_rope_inputs(g)
    t, h = g["t"], g["h"]
    q, k, v = x, x.flip(0)[:, :1].contiguous(), (x * 0.5)[:, :1].contiguous()
    kc = torch.zeros(2, 256, 1, 128, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    slots = torch.tensor([5, 6, 300, -1, 8, 511, 0], dtype=torch.int32)
    qn = oracle.qk_norm_rope_append(q, k, v, weight, weight, g["eps"], positions, cache, kc, vc, slots)
    want = torch.from_numpy(np.load(GOLD / "norm_rope_out.npy")).view(torch.bfloat16)
    assert torch.equal(qn.view(torch.int16), want.view(torch.int16))
    keep = slots >= 0
    assert torch.equal(vc.view(-1, 1, 128)[slots[keep].long()], v[keep])
    assert int((kc.view(-1, 128).abs().sum(-1) > 0).sum()) == int(keep.sum())
