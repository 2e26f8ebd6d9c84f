"""Paged chunked-prefill attention and the dense causal op against the CPU oracle."""
from pathlib import Path

import numpy as np
import pytest
import torch

from gpu_util import ATOL_BF16, RTOL_BF16, assert_close, to_dev
from infer_b200 import ops, selftest, workloads
from oracle import paged_kv_oracle as oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(params=[1, 0], ids=["mma", "tcgen05"], autouse=True)
def prefill_kernel(request):
    """Every test of this file runs on both prefill kernels: the tcgen05 kernel through the
    regular entry points, the mma.sync cross-check kernel through the self-test ones."""
    if request.param == 0:
        yield 0
    else:
        with selftest.variant(prefill_kernel=1):
            yield 1


def _run(w):
    d = to_dev(w)
    cu_q, cu_k = w.cu_seqlens()
    ops.store_kvcache(d["k"], d["v"], d["k_cache"], d["v_cache"], d["slot_mapping"])
    got = ops.paged_attn_prefill(d["q"], d["k_cache"], d["v_cache"], cu_q.cuda(), cu_k.cuda(), max(w.new_lens),
                                 max(w.context_lens), w.scale, d["block_tables"])
    torch.cuda.synchronize()
    kc, vc = w.k_cache.clone(), w.v_cache.clone()
    oracle.store_kvcache(w.k, w.v, kc, vc, w.slot_mapping)
    want = oracle.paged_prefill(w.q, kc, vc, cu_q, cu_k, w.block_tables_tensor(), w.scale)
    return got, want, d


def test_prefill_chunked_reduced():
    got, want, _ = _run(workloads.config2(n_seqs=4, max_prefix=700, chunk=300))
    assert_close(got, want, ATOL_BF16, RTOL_BF16, "chunked prefill 4x300")


def test_prefill_ragged_chunks_and_no_prefix():
    """Chunk lengths that are not multiples of the tile, one sequence without any prefix,
    one with a prefix ending exactly on a page boundary."""
    w = workloads.config2(n_seqs=5, max_prefix=600, chunk=130, seed=31)
    # rebuild with ragged chunk lengths on the same page lists
    from infer_b200.metadata import chunk_slots
    prefixes = [0, 256, 1, 511, 300]
    chunks = [130, 64, 1, 77, 200]
    gen = torch.Generator().manual_seed(31)
    lens = [p + c for p, c in zip(prefixes, chunks)]
    perm = torch.randperm(w.num_blocks, generator=gen).tolist()
    tables, at = [], 0
    for n in lens:
        need = -(-n // 256)
        tables.append(perm[at:at + need])
        at += need
    slots = [s for t, p, n in zip(tables, prefixes, lens) for s in chunk_slots(t, p, n, 256)]
    tq = sum(chunks)
    w.block_tables, w.context_lens, w.new_lens = tables, lens, chunks
    w.slot_mapping = torch.tensor(slots, dtype=torch.int32)
    w.q = torch.randn(tq, 16, 128, generator=gen).bfloat16()
    w.k = torch.randn(tq, 8, 128, generator=gen).bfloat16()
    w.v = torch.randn(tq, 8, 128, generator=gen).bfloat16()
    got, want, _ = _run(w)
    assert_close(got, want, ATOL_BF16, RTOL_BF16, "ragged prefill")


def test_prefill_odd_group_size():
    """Three query heads per KV head: the two query tiles of a thread block are then two row
    blocks of one head with different numbers of key tiles (the other tests pair two heads)."""
    w = workloads.config2(n_seqs=3, max_prefix=900, chunk=420, seed=35)
    gen = torch.Generator().manual_seed(35)
    w.q = torch.randn(w.q.shape[0], 24, 128, generator=gen).bfloat16()
    w.n_q_heads = 24
    got, want, _ = _run(w)
    assert_close(got, want, ATOL_BF16, RTOL_BF16, "prefill, group 3")


def test_prefill_full_size_against_oracle(prefill_kernel):
    """The benchmark configuration itself (16 sequences, prefix up to 4096, chunk 2048).  Two whole
    sequences - the one with the longest prefix (48 key tiles per row, thousands of keys through
    the lazy rescale) and the one with the shortest - are compared with the CPU oracle, which only
    needs those sequences' pages; the mma.sync kernel, an independent program, must agree with the
    tcgen05 kernel on every row; and the last row of every chunk must equal the decode kernel's
    answer for that position."""
    if prefill_kernel != 0:
        pytest.skip("one run covers both kernels")
    w = workloads.config2(device="cuda")
    cu_q, cu_k = (t.cuda() for t in w.cu_seqlens())
    bt = w.block_tables_tensor().cuda()
    ops.store_kvcache(w.k, w.v, w.k_cache, w.v_cache, w.slot_mapping.cuda())
    args = (w.q, w.k_cache, w.v_cache, cu_q, cu_k, max(w.new_lens), max(w.context_lens), w.scale, bt)
    got = ops.paged_attn_prefill(*args)
    with selftest.variant(prefill_kernel=1):
        other = ops.paged_attn_prefill(*args)
    torch.cuda.synchronize()
    assert_close(got, other, ATOL_BF16, RTOL_BF16, "tcgen05 vs mma.sync, full size")
    order = np.argsort(w.context_lens)
    cu = cu_q.cpu()
    for b in (int(order[-1]), int(order[0])):
        pages = torch.tensor(w.block_tables[b])
        kc, vc = w.k_cache[pages.cuda()].cpu(), w.v_cache[pages.cuda()].cpu()
        rows = slice(int(cu[b]), int(cu[b + 1]))
        n_new, n_ctx = w.new_lens[b], w.context_lens[b]
        want = oracle.paged_prefill(w.q[rows].cpu(), kc, vc, torch.tensor([0, n_new], dtype=torch.int32),
                                    torch.tensor([0, n_ctx], dtype=torch.int32),
                                    torch.arange(len(pages), dtype=torch.int32)[None], w.scale)
        assert_close(got[rows], want, ATOL_BF16, RTOL_BF16, f"full-size prefill seq {b} (ctx {n_ctx}) vs oracle")
    last = (cu_q[1:] - 1).long()
    dec = ops.paged_attn_decode(w.q[last].contiguous(), w.k_cache, w.v_cache,
                                torch.tensor(w.context_lens, dtype=torch.int32, device="cuda"), bt, w.scale)
    assert_close(got[last], dec, ATOL_BF16, RTOL_BF16, "last chunk rows vs decode, full size")


def test_prefill_last_row_equals_decode():
    w = workloads.config2(n_seqs=3, max_prefix=900, chunk=200, seed=33)
    got, _, d = _run(w)
    cu_q, _ = w.cu_seqlens()
    last = (cu_q[1:] - 1).long()
    dec = ops.paged_attn_decode(d["q"][last.cuda()].contiguous(), d["k_cache"], d["v_cache"],
                                torch.tensor(w.context_lens, dtype=torch.int32, device="cuda"), d["block_tables"], w.scale)
    assert_close(got[last.cuda()], dec, ATOL_BF16, RTOL_BF16, "last chunk row vs decode")


def test_dense_flash_attn_prefill_golden(golden):
    """The reference's own test case for this op (test/op.py:269-287) at reduced head count,
    against the SDPA output stored in the golden fixture, with the reference's tolerance."""
    g = golden["attention"]
    gen = torch.Generator().manual_seed(g["seed"])
    Q = torch.randn(1, 4, 64, 128, generator=gen).bfloat16().cuda()
    K = torch.randn(1, 4, 64, 128, generator=gen).bfloat16().cuda()
    V = torch.randn(1, 4, 64, 128, generator=gen).bfloat16().cuda()
    O = torch.empty_like(Q)
    ops.flash_attn_prefill(Q, K, V, O)
    want = torch.from_numpy(np.load(Path(__file__).parent / "golden" / "dense_causal_O.npy")).view(torch.bfloat16)
    assert_close(O, want, 2e-2, 1e-3, "dense causal golden")


@pytest.mark.parametrize("shape", [(1, 32, 32, 64), (2, 8, 2, 200), (1, 4, 4, 1000)])
def test_dense_flash_attn_prefill_shapes(shape):
    b, hq, hkv, s = shape
    gen = torch.Generator().manual_seed(s)
    Q = torch.randn(b, hq, s, 128, generator=gen).bfloat16()
    K = torch.randn(b, hkv, s, 128, generator=gen).bfloat16()
    V = torch.randn(b, hkv, s, 128, generator=gen).bfloat16()
    O = torch.empty_like(Q).cuda()
    ops.flash_attn_prefill(Q.cuda(), K.cuda(), V.cuda(), O)
    assert_close(O, oracle.dense_causal(Q, K, V), ATOL_BF16, RTOL_BF16, f"dense {shape}")


def test_torch_ops_namespace():
    """The ops are reachable as torch.ops._C.* with the reference's out-parameter style."""
    from infer_b200 import infer_ops
    Q = torch.randn(1, 2, 64, 128, device="cuda").bfloat16()
    O1, O2 = torch.empty_like(Q), torch.empty_like(Q)
    infer_ops.flash_attn_prefill(Q, Q, Q, O1)
    torch.ops._C.flash_attn_prefill(Q, Q, Q, O2)
    assert torch.equal(O1, O2)
    assert_close(O1, oracle.dense_causal(Q.cpu(), Q.cpu(), Q.cpu()), ATOL_BF16, RTOL_BF16, "torch.ops._C")
