"""Paged decode attention through the C ABI against the CPU oracle (bf16 pools)."""
import numpy as np
import pytest
import torch

from gpu_util import ATOL_BF16, RTOL_BF16, assert_close, to_dev
from infer_b200 import ops, selftest, workloads
from oracle import paged_kv_oracle as oracle

pytestmark = pytest.mark.gpu

VARIANTS = [0, 1, 2, 4, 8]   # kv heads per tile: 0 = the regular entry point (one head), others through the self-test call


def _decode(hpc, *args, **kw):
    if hpc == 0:
        return ops.paged_attn_decode(*args, **kw)
    with selftest.variant(decode_heads_per_tile=hpc):
        return ops.paged_attn_decode(*args, **kw)


def _step(w, hpc=0):
    """append + decode on the GPU, the same two calls on the oracle."""
    d = to_dev(w)
    ops.store_kvcache(d["k"], d["v"], d["k_cache"], d["v_cache"], d["slot_mapping"])
    got = _decode(hpc, d["q"], d["k_cache"], d["v_cache"], d["context_lens"], d["block_tables"], w.scale)
    torch.cuda.synchronize()
    kc, vc = w.k_cache.clone(), w.v_cache.clone()
    oracle.store_kvcache(w.k, w.v, kc, vc, w.slot_mapping)
    want = oracle.paged_decode(w.q, kc, vc, w.context_lens_tensor(), w.block_tables_tensor(), w.scale)
    return got, want


@pytest.mark.parametrize("hpc", VARIANTS)
def test_decode_config0(hpc):
    got, want = _step(workloads.config0(), hpc)
    assert_close(got, want, ATOL_BF16, RTOL_BF16, f"config0 hpc={hpc}")


@pytest.mark.parametrize("hpc", VARIANTS)
def test_decode_qwen3_8b_shape_reduced(hpc):
    got, want = _step(workloads.config1(batch=12, lo=200, hi=3000), hpc)
    assert_close(got, want, ATOL_BF16, RTOL_BF16, f"config1/12 hpc={hpc}")


@pytest.mark.parametrize("hpc", [0, 2, 8])
def test_decode_group8_shared_prefix_reduced(hpc):
    w = workloads.config4(batch=16, cap=3000)
    got, want = _step(w, hpc)
    assert_close(got, want, ATOL_BF16, RTOL_BF16, f"config4/16 hpc={hpc}")


@pytest.mark.parametrize("hq,hkv", [(24, 8), (40, 8), (12, 2), (7, 1), (48, 8)])
@pytest.mark.parametrize("hpc", [0, 2])
def test_decode_any_group_size(hq, hkv, hpc):
    """Query-head groups that are not a power of two (3, 5, 6, 7): the reference's decode call
    (flash_attn_with_kvcache, infer/ops/attention.py:118-120) takes any Hq % Hkv == 0, and
    Qwen3-14B is 40 query heads over 8 KV heads."""
    if hkv % max(hpc, 1):
        pytest.skip("heads per tile must divide the kv heads")
    rng = np.random.default_rng(hq)
    lens = rng.integers(100, 2600, size=10)
    w = workloads._decode_workload("any-group", 77 + hq, hq, hkv, lens, workloads._pool_size(lens), "cpu")
    got, want = _step(w, hpc)
    assert_close(got, want, ATOL_BF16, RTOL_BF16, f"{hq}q/{hkv}kv hpc={hpc}")


@pytest.mark.parametrize("world", [2, 4, 8])
def test_decode_head_shards_match_full(world):
    """Each KV-head shard computed on its own equals the matching slice of the oracle."""
    w = workloads.config0()
    kc, vc = w.k_cache.clone(), w.v_cache.clone()
    oracle.store_kvcache(w.k, w.v, kc, vc, w.slot_mapping)
    want = oracle.paged_decode(w.q, kc, vc, w.context_lens_tensor(), w.block_tables_tensor(), w.scale)
    per = w.n_q_heads // world
    for r in (0, world - 1):
        got, _ = _step(w.shard(r, world))
        assert_close(got, want[:, r * per:(r + 1) * per], ATOL_BF16, RTOL_BF16, f"shard {r}/{world}")


@pytest.mark.parametrize("hpc", VARIANTS)
def test_decode_edge_lengths(hpc):
    """Lengths around tile and page boundaries, an empty row, -1 padding, stale pool bytes."""
    lens = [1, 15, 16, 17, 0, 127, 128, 129, 255, 256, 257, 511, 513, 1]
    hq, hkv = 16, 8
    gen = torch.Generator().manual_seed(21)
    num_blocks = 40
    kc = torch.randn(num_blocks, 256, hkv, 128, generator=gen).bfloat16()
    vc = torch.randn(num_blocks, 256, hkv, 128, generator=gen).bfloat16()
    # rows that no sequence owns hold NaN patterns: nothing past a context may leak in
    perm = torch.randperm(num_blocks, generator=gen).tolist()
    tables, at = [], 0
    owned = torch.zeros(num_blocks * 256, dtype=torch.bool)
    for n in lens:
        need = -(-n // 256)
        pages = perm[at:at + need]
        at += need
        tables.append(pages + [-1] * (4 - need))
        for i, pg in enumerate(pages):
            owned[pg * 256: pg * 256 + min(256, n - i * 256)] = True
    kc.view(-1, hkv, 128)[~owned] = float("nan")
    vc.view(-1, hkv, 128)[~owned] = float("nan")
    q = torch.randn(len(lens), hq, 128, generator=gen).bfloat16()
    bt = torch.tensor(tables, dtype=torch.int32)
    cl = torch.tensor(lens, dtype=torch.int32)
    out = torch.full((len(lens), hq, 128), 7.0, dtype=torch.bfloat16, device="cuda")
    _decode(hpc, q.cuda(), kc.cuda(), vc.cuda(), cl.cuda(), bt.cuda(), 0.09, out=out)
    torch.cuda.synchronize()
    want = oracle.paged_decode(q, kc, vc, cl, bt, 0.09)
    live = cl > 0
    assert_close(out[live.cuda()], want[live], ATOL_BF16, RTOL_BF16, f"edges hpc={hpc}")
    assert bool((out[~live.cuda()] == 7.0).all()), "row with context_len == 0 was written"


def test_decode_golden_sdpa(golden):
    """The SDPA expectations of the golden fixture, keys laid out in scattered pages."""
    from infer_b200 import metadata
    g = golden["attention"]
    gen = torch.Generator().manual_seed(g["seed"])
    for _ in range(3):
        torch.randn(1, 4, 64, 128, generator=gen)
    lens, hq, hkv = g["decode_lens"], g["decode_hq"], g["decode_hkv"]
    want = torch.from_numpy(np.load(__import__("pathlib").Path(__file__).parent / "golden" / "decode_sdpa_O.npy"))
    kc = torch.zeros(16, 256, hkv, 128, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    perm = torch.randperm(16, generator=torch.Generator().manual_seed(1)).tolist()
    tables, qs, at = [], [], 0
    for n in lens:
        q = torch.randn(hq, 1, 128, generator=gen).bfloat16()
        k = torch.randn(hkv, n, 128, generator=gen).bfloat16()
        v = torch.randn(hkv, n, 128, generator=gen).bfloat16()
        pages = perm[at:at + -(-n // 256)]
        at += len(pages)
        slots = torch.tensor(metadata.chunk_slots(pages, 0, n, 256), dtype=torch.int32, device="cuda")
        ops.store_kvcache(k.transpose(0, 1).contiguous().cuda(), v.transpose(0, 1).contiguous().cuda(), kc, vc, slots)
        tables.append(pages + [-1] * (3 - len(pages)))
        qs.append(q[:, 0, :])
    got = ops.paged_attn_decode(torch.stack(qs).cuda(), kc, vc, torch.tensor(lens, dtype=torch.int32, device="cuda"),
                                torch.tensor(tables, dtype=torch.int32, device="cuda"), 128 ** -0.5)
    assert_close(got, want, ATOL_BF16, RTOL_BF16, "golden sdpa")


def test_decode_full_size_subset_against_oracle():
    """Config 2 at full size (64 sequences, ~1.2 GB of KV): every row finite; three
    sequences (shortest, longest, one in between) checked against the oracle, which only
    needs those sequences' pages on the CPU."""
    w = workloads.config1(device="cuda")
    cl = w.context_lens_tensor().cuda()
    bt = w.block_tables_tensor().cuda()
    slots = w.slot_mapping.cuda()
    ops.store_kvcache(w.k, w.v, w.k_cache, w.v_cache, slots)
    got = ops.paged_attn_decode(w.q, w.k_cache, w.v_cache, cl, bt, w.scale)
    torch.cuda.synchronize()
    assert torch.isfinite(got.float()).all()
    order = np.argsort(w.context_lens)
    for b in (int(order[0]), int(order[len(order) // 2]), int(order[-1])):
        pages = torch.tensor(w.block_tables[b])
        kc = w.k_cache[pages.cuda()].cpu()
        vc = w.v_cache[pages.cuda()].cpu()
        local = torch.arange(len(pages), dtype=torch.int32)[None]
        want = oracle.paged_decode(w.q[b:b + 1].cpu(), kc, vc, torch.tensor([w.context_lens[b]], dtype=torch.int32),
                                   local, w.scale)
        assert_close(got[b:b + 1], want, ATOL_BF16, RTOL_BF16, f"full-size seq {b} (len {w.context_lens[b]})")


def test_decode_in_cuda_graph():
    """append + decode captured once and replayed with new metadata in the static buffers,
    the way the reference replays its decode graphs (infer/engine/model_runner.py:135-152)."""
    w = workloads.config0()
    d = to_dev(w)
    width = 8
    bt_static = torch.zeros(w.batch, width, dtype=torch.int32, device="cuda")
    bt_static[:, :d["block_tables"].shape[1]] = d["block_tables"]
    out = torch.zeros_like(d["q"])
    # eager warm-up (allocates scratch, creates the pool handle)
    ops.store_kvcache(d["k"], d["v"], d["k_cache"], d["v_cache"], d["slot_mapping"])
    ops.paged_attn_decode(d["q"], d["k_cache"], d["v_cache"], d["context_lens"], bt_static, w.scale, out=out)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ops.store_kvcache(d["k"], d["v"], d["k_cache"], d["v_cache"], d["slot_mapping"])
        ops.paged_attn_decode(d["q"], d["k_cache"], d["v_cache"], d["context_lens"], bt_static, w.scale, out=out)
    # replay on different lengths: shorten every context by 10 tokens
    new_lens = [max(1, n - 10) for n in w.context_lens]
    new_slots = [t[(n - 1) // 256] * 256 + (n - 1) % 256 for t, n in zip(w.block_tables, new_lens)]
    d["context_lens"].copy_(torch.tensor(new_lens, dtype=torch.int32))
    d["slot_mapping"].copy_(torch.tensor(new_slots, dtype=torch.int32))
    out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    kc, vc = w.k_cache.clone(), w.v_cache.clone()
    oracle.store_kvcache(w.k, w.v, kc, vc, w.slot_mapping)
    oracle.store_kvcache(w.k, w.v, kc, vc, torch.tensor(new_slots, dtype=torch.int32))
    want = oracle.paged_decode(w.q, kc, vc, torch.tensor(new_lens, dtype=torch.int32), w.block_tables_tensor(), w.scale)
    assert_close(out, want, ATOL_BF16, RTOL_BF16, "graph replay")


def _oracle_rows(w, got, rows, what):
    """Compare the given sequences of a GPU-resident workload with the oracle, which only needs
    those sequences' pages on the CPU."""
    for b in rows:
        pages = torch.tensor(w.block_tables[b])
        kc, vc = w.k_cache[pages.cuda()].cpu(), w.v_cache[pages.cuda()].cpu()
        local = torch.arange(len(pages), dtype=torch.int32)[None]
        want = oracle.paged_decode(w.q[b:b + 1].cpu(), kc, vc, torch.tensor([w.context_lens[b]], dtype=torch.int32),
                                   local, w.scale)
        assert_close(got[b:b + 1], want, ATOL_BF16, RTOL_BF16, f"{what} seq {b} (len {w.context_lens[b]})")


def test_decode_long_context_full_size_against_oracle():
    """The long-context configuration at full size on one GPU (batch 256, 64q/8kv heads, contexts up
    to 32768 = 128 pages, half the batch sharing the pages of a 2048-token prefix): the longest
    sequence (its (sequence, head) rows span many thread blocks and go through the ticketed merge),
    two sequences of the shared-prefix half, the shortest and a median one against the oracle."""
    w = workloads.config4(device="cuda", longest_at_cap=True)
    assert max(w.context_lens) == 32768
    cl, bt = w.context_lens_tensor().cuda(), w.block_tables_tensor().cuda()
    ops.store_kvcache(w.k, w.v, w.k_cache, w.v_cache, w.slot_mapping.cuda())
    got = ops.paged_attn_decode(w.q, w.k_cache, w.v_cache, cl, bt, w.scale)
    torch.cuda.synchronize()
    assert torch.isfinite(got.float()).all()
    order = np.argsort(w.context_lens)
    shared = [b for b in range(w.batch // 2)]
    rows = {int(order[-1]), int(order[0]), int(order[len(order) // 2]), shared[0], shared[-1]}
    assert w.block_tables[shared[0]][:8] == w.block_tables[shared[-1]][:8]      # the prefix pages really are shared
    _oracle_rows(w, got, sorted(rows), "long-context full size")
    # a second pass over the same scratch must give the same bits (tickets were left at zero)
    again = ops.paged_attn_decode(w.q, w.k_cache, w.v_cache, cl, bt, w.scale)
    torch.cuda.synchronize()
    assert torch.equal(got, again)


def test_decode_steps_chained_without_host_sync():
    """advance -> append -> decode, step after step on one stream with no host synchronisation in
    between, across a page boundary: the attention kernel's prologue reads context_lens while the
    kernels in front may still be in flight (programmatic dependent launch), so every step's result
    depends on the launches being ordered correctly."""
    from infer_b200.metadata import DecodeState
    from infer_b200.sequence import Sequence
    hq, hkv, nb, steps = 16, 8, 24, 24
    gen = torch.Generator().manual_seed(5)
    start = [250, 255, 3, 511, 256, 100]                      # several rows cross into a new page within the steps
    kc = torch.randn(nb, 256, hkv, 128, generator=gen).bfloat16()
    vc = torch.randn(nb, 256, hkv, 128, generator=gen).bfloat16()
    perm = torch.randperm(nb, generator=gen).tolist()
    seqs, at = [], 0
    for n in start:
        s = Sequence(list(range(n)))
        need = -(-(n + steps) // 256)
        s.block_table = perm[at:at + need]
        at += need
        seqs.append(s)
    state = DecodeState(len(start), 4, 256, "cuda")
    state.load(seqs)
    qs = torch.randn(steps, len(start), hq, 128, generator=gen).bfloat16()
    ks = torch.randn(steps, len(start), hkv, 128, generator=gen).bfloat16()
    vs = torch.randn(steps, len(start), hkv, 128, generator=gen).bfloat16()
    dq, dk, dv, dkc, dvc = qs.cuda(), ks.cuda(), vs.cuda(), kc.cuda(), vc.cuda()
    outs = torch.zeros(steps, len(start), hq, 128, dtype=torch.bfloat16, device="cuda")
    ops.paged_attn_decode(dq[0], dkc, dvc, torch.ones(len(start), dtype=torch.int32, device="cuda"),
                          state.block_tables, 0.09)           # sizes the scratch before the chain
    torch.cuda.synchronize()
    for t in range(steps):
        state.advance()
        ops.store_kvcache(dk[t], dv[t], dkc, dvc, state.slot_mapping)
        ops.paged_attn_decode(dq[t], dkc, dvc, state.context_lens, state.block_tables, 0.09, out=outs[t])
    torch.cuda.synchronize()
    lens = list(start)
    bt = torch.tensor([s.block_table + [-1] * (4 - len(s.block_table)) for s in seqs], dtype=torch.int32)
    for t in range(steps):
        lens = [n + 1 for n in lens]
        slots = torch.tensor([s.block_table[(n - 1) // 256] * 256 + (n - 1) % 256 for s, n in zip(seqs, lens)],
                             dtype=torch.int32)
        oracle.store_kvcache(ks[t], vs[t], kc, vc, slots)
        want = oracle.paged_decode(qs[t], kc, vc, torch.tensor(lens, dtype=torch.int32), bt, 0.09)
        assert_close(outs[t], want, ATOL_BF16, RTOL_BF16, f"chained step {t}")
    assert torch.equal(dkc.cpu().view(torch.int16), kc.view(torch.int16))


def test_decode_rejects_bad_arguments():
    kc = torch.zeros(2, 256, 8, 128, dtype=torch.bfloat16, device="cuda")
    q = torch.zeros(1, 72, 128, dtype=torch.bfloat16, device="cuda")       # 72 % 8 == 0 but 9 query heads per kv head
    cl = torch.ones(1, dtype=torch.int32, device="cuda")
    bt = torch.zeros(1, 1, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="geometry"):
        ops.paged_attn_decode(q, kc, kc, cl, bt, 0.1)
    with pytest.raises(RuntimeError):
        ops.paged_attn_decode(q[:, :16].contiguous(), kc, kc, cl.long(), bt, 0.1)


def test_decode_reads_q_from_and_writes_out_to_pinned_host_memory():
    """A host-fed step can skip two copies: q stays in pinned host memory and the kernel writes the output rows
    straight into a pinned host tensor; the bits equal those of the all-device call."""
    w = workloads.config1(batch=12, lo=200, hi=3000)
    d = to_dev(w)
    want = ops.paged_attn_decode(d["q"], d["k_cache"], d["v_cache"], d["context_lens"], d["block_tables"], w.scale)
    q_host = w.q.clone().pin_memory()
    out_host = torch.zeros(w.q.shape, dtype=torch.bfloat16).pin_memory()
    ops.paged_attn_decode(q_host, d["k_cache"], d["v_cache"], d["context_lens"], d["block_tables"], w.scale, out=out_host)
    torch.cuda.synchronize()
    assert torch.equal(out_host, want.cpu())
    with pytest.raises(RuntimeError, match="pinned"):
        ops.paged_attn_decode(w.q, d["k_cache"], d["v_cache"], d["context_lens"], d["block_tables"], w.scale, out=out_host)


def _fused_step(w, strided=False):
    """One decode step through the fused op, against oracle append + oracle decode."""
    d = to_dev(w)
    if strided:          # k and v as column slices of a wider row, the way they come out of a fused qkv projection
        hkv = w.n_kv_heads
        wide = torch.zeros(w.batch, 3 * hkv * 128 + 64, dtype=torch.bfloat16, device="cuda")
        wide[:, 64:64 + hkv * 128] = d["k"].reshape(w.batch, -1)
        wide[:, 64 + hkv * 128:64 + 2 * hkv * 128] = d["v"].reshape(w.batch, -1)
        k = wide[:, 64:64 + hkv * 128].view(w.batch, hkv, 128)
        v = wide[:, 64 + hkv * 128:64 + 2 * hkv * 128].view(w.batch, hkv, 128)
    else:
        k, v = d["k"], d["v"]
    got = ops.paged_attn_decode_append(d["q"], k, v, d["k_cache"], d["v_cache"], d["context_lens"], d["block_tables"], w.scale)
    torch.cuda.synchronize()
    kc, vc = w.k_cache.clone(), w.v_cache.clone()
    oracle.store_kvcache(w.k, w.v, kc, vc, w.slot_mapping)
    want = oracle.paged_decode(w.q, kc, vc, w.context_lens_tensor(), w.block_tables_tensor(), w.scale)
    assert torch.equal(d["k_cache"].cpu().view(torch.int16), kc.view(torch.int16)), "k pool differs from the oracle's append"
    assert torch.equal(d["v_cache"].cpu().view(torch.int16), vc.view(torch.int16)), "v pool differs from the oracle's append"
    return got, want


@pytest.mark.parametrize("strided", [False, True])
def test_fused_append_decode_matches_oracle(strided):
    """store_kvcache + paged_attn_decode in one launch (infer/ops/attention.py:109 and :117-121): pools bit-exact,
    outputs within tolerance; the shared-prefix workload has far more sequences ending in a CTA's range than
    the sixteen the appending lanes look up at a time."""
    for w in (workloads.config0(), workloads.config1(batch=12, lo=200, hi=3000), workloads.config4(batch=16, cap=3000)):
        got, want = _fused_step(w, strided)
        assert_close(got, want, ATOL_BF16, RTOL_BF16, f"fused append + decode, {w.name}")


def test_fused_append_decode_many_short_sequences():
    """700 sequences of 1 to 300 tokens: dozens of sequences end inside every CTA's range."""
    gen = torch.Generator().manual_seed(700)
    b, hq, hkv = 700, 8, 2
    lens = torch.randint(1, 301, (b,), generator=gen)
    nb = int((-(-lens // 256)).sum()) + 3
    kc = torch.randn(nb, 256, hkv, 128, generator=gen).bfloat16()
    vc = torch.randn(nb, 256, hkv, 128, generator=gen).bfloat16()
    perm = torch.randperm(nb, generator=gen).tolist()
    bt = torch.full((b, 2), -1, dtype=torch.int32)
    at = 0
    for i, n in enumerate(lens.tolist()):
        for j in range(-(-n // 256)):
            bt[i, j] = perm[at]
            at += 1
    slots = torch.tensor([int(bt[i, (n - 1) // 256]) * 256 + (n - 1) % 256 for i, n in enumerate(lens.tolist())], dtype=torch.int32)
    q = torch.randn(b, hq, 128, generator=gen).bfloat16()
    k = torch.randn(b, hkv, 128, generator=gen).bfloat16()
    v = torch.randn(b, hkv, 128, generator=gen).bfloat16()
    cl = lens.to(torch.int32)
    dkc, dvc = kc.cuda(), vc.cuda()
    got = ops.paged_attn_decode_append(q.cuda(), k.cuda(), v.cuda(), dkc, dvc, cl.cuda(), bt.cuda(), 0.09)
    torch.cuda.synchronize()
    oracle.store_kvcache(k, v, kc, vc, slots)
    assert torch.equal(dkc.cpu().view(torch.int16), kc.view(torch.int16)) and torch.equal(dvc.cpu().view(torch.int16), vc.view(torch.int16))
    want = oracle.paged_decode(q, kc, vc, cl, bt, 0.09)
    assert_close(got, want, ATOL_BF16, RTOL_BF16, "fused step, 700 short sequences")


def test_fused_append_decode_edge_lengths_and_stale_rows():
    """The appended token alone in its sequence, alone on a fresh page, at tile and page ends; an empty row;
    every slot no sequence owns - the new tokens' slots included - holds NaN patterns before the call."""
    lens = [1, 2, 128, 129, 256, 257, 0, 513, 1, 300]
    hq, hkv, nb = 16, 8, 40
    gen = torch.Generator().manual_seed(77)
    kc = torch.randn(nb, 256, hkv, 128, generator=gen).bfloat16()
    vc = torch.randn(nb, 256, hkv, 128, generator=gen).bfloat16()
    perm = torch.randperm(nb, generator=gen).tolist()
    tables, slots, at = [], [], 0
    owned = torch.zeros(nb * 256, dtype=torch.bool)
    for n in lens:
        need = -(-n // 256)
        pages = perm[at:at + need]
        at += need
        tables.append(pages + [-1] * (4 - need))
        for pos in range(n - 1):                       # the rows that exist before the step
            owned[pages[pos // 256] * 256 + pos % 256] = True
        slots.append(pages[(n - 1) // 256] * 256 + (n - 1) % 256 if n > 0 else -1)
    kc.view(-1, hkv, 128)[~owned] = float("nan")
    vc.view(-1, hkv, 128)[~owned] = float("nan")
    q = torch.randn(len(lens), hq, 128, generator=gen).bfloat16()
    k = torch.randn(len(lens), hkv, 128, generator=gen).bfloat16()
    v = torch.randn(len(lens), hkv, 128, generator=gen).bfloat16()
    bt, cl = torch.tensor(tables, dtype=torch.int32), torch.tensor(lens, dtype=torch.int32)
    dkc, dvc = kc.cuda(), vc.cuda()
    out = torch.full((len(lens), hq, 128), 7.0, dtype=torch.bfloat16, device="cuda")
    ops.paged_attn_decode_append(q.cuda(), k.cuda(), v.cuda(), dkc, dvc, cl.cuda(), bt.cuda(), 0.09, out=out)
    torch.cuda.synchronize()
    oracle.store_kvcache(k, v, kc, vc, torch.tensor(slots, dtype=torch.int32))
    assert torch.equal(dkc.cpu().view(torch.int16), kc.view(torch.int16)) and torch.equal(dvc.cpu().view(torch.int16), vc.view(torch.int16))
    want = oracle.paged_decode(q, kc, vc, cl, bt, 0.09)
    live = cl > 0
    assert_close(out[live.cuda()], want[live], ATOL_BF16, RTOL_BF16, "fused step, edge lengths")
    assert bool((out[~live.cuda()] == 7.0).all())


def test_fused_append_decode_in_cuda_graph_over_steps():
    """The fused step captured once and replayed for 20 steps, lengths advanced on the device between replays
    (DecodeState) by the kernel directly in front of it, new rows written into static buffers: pools and outputs
    follow the oracle step by step, across page boundaries."""
    from infer_b200.metadata import DecodeState
    from infer_b200.sequence import Sequence
    hq, hkv, nb, steps = 16, 8, 16, 20
    gen = torch.Generator().manual_seed(9)
    start = [250, 255, 3, 100]
    kc = torch.randn(nb, 256, hkv, 128, generator=gen).bfloat16()
    vc = torch.randn(nb, 256, hkv, 128, generator=gen).bfloat16()
    perm = torch.randperm(nb, generator=gen).tolist()
    seqs, at = [], 0
    for n in start:
        s = Sequence(list(range(n)))
        need = -(-(n + steps) // 256)
        s.block_table = perm[at:at + need]
        at += need
        seqs.append(s)
    state = DecodeState(len(start), 3, 256, "cuda")
    state.load(seqs)
    dq = torch.zeros(len(start), hq, 128, dtype=torch.bfloat16, device="cuda")
    dk = torch.zeros(len(start), hkv, 128, dtype=torch.bfloat16, device="cuda")
    dv = torch.zeros_like(dk)
    out = torch.zeros_like(dq)
    dkc, dvc = kc.cuda(), vc.cuda()
    ops.paged_attn_decode(dq, dkc, dvc, torch.ones(len(start), dtype=torch.int32, device="cuda"), state.block_tables, 0.09)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        state.advance()
        ops.paged_attn_decode_append(dq, dk, dv, dkc, dvc, state.context_lens, state.block_tables, 0.09, out=out)
    state.load(seqs)                                       # capture launches nothing: lengths are still the start lengths
    torch.cuda.synchronize()
    lens = list(start)
    bt = torch.tensor([s.block_table + [-1] * (3 - len(s.block_table)) for s in seqs], dtype=torch.int32)
    for t in range(steps):
        q = torch.randn(len(start), hq, 128, generator=gen).bfloat16()
        k = torch.randn(len(start), hkv, 128, generator=gen).bfloat16()
        v = torch.randn(len(start), hkv, 128, generator=gen).bfloat16()
        dq.copy_(q); dk.copy_(k); dv.copy_(v)
        graph.replay()
        torch.cuda.synchronize()
        lens = [n + 1 for n in lens]
        slots = torch.tensor([s.block_table[(n - 1) // 256] * 256 + (n - 1) % 256 for s, n in zip(seqs, lens)], dtype=torch.int32)
        oracle.store_kvcache(k, v, kc, vc, slots)
        want = oracle.paged_decode(q, kc, vc, torch.tensor(lens, dtype=torch.int32), bt, 0.09)
        assert_close(out, want, ATOL_BF16, RTOL_BF16, f"fused step {t} in a graph")
    assert torch.equal(dkc.cpu().view(torch.int16), kc.view(torch.int16)) and torch.equal(dvc.cpu().view(torch.int16), vc.view(torch.int16))


def test_fused_append_decode_rejects_e4m3_pools():
    """Through the C ABI: an e4m3 pool handle is turned down with INFER_ERR_DTYPE before anything is launched."""
    import ctypes as C
    from infer_b200 import _lib
    k8 = torch.zeros(4, 256, 2, 128, dtype=torch.uint8, device="cuda")
    v8 = torch.zeros_like(k8)
    ks = torch.zeros(4, 2, device="cuda")
    vs = torch.zeros_like(ks)
    pool = ops.pool_of(k8, v8, ks, vs)
    q = torch.zeros(1, 4, 128, dtype=torch.bfloat16, device="cuda")
    kv = torch.zeros(1, 2, 128, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros_like(q)
    cl = torch.ones(1, dtype=torch.int32, device="cuda")
    bt = torch.zeros(1, 1, dtype=torch.int32, device="cuda")
    ws = torch.zeros(pool.decode_workspace_bytes(1, 4), dtype=torch.uint8, device="cuda")
    p = lambda t: C.c_void_p(t.data_ptr())
    rc = _lib.load().infer_paged_decode_append(pool.handle, p(out), p(q), p(kv), p(kv), 256, 256, p(cl), p(bt), 1, 1, 4,
                                               0.09, p(ws), ws.numel(), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == _lib.ERR_DTYPE
    torch.cuda.synchronize()
    assert bool((k8 == 0).all())


def test_fused_append_decode_rows_and_output_in_pinned_host_memory():
    """q, the new k and v rows and the output in pinned host memory (the kernel reads and writes them over PCIe):
    the same pools and rows as with device tensors."""
    w = workloads.config1(batch=12, lo=200, hi=3000)
    d = to_dev(w)
    q_h, k_h, v_h = w.q.clone().pin_memory(), w.k.clone().pin_memory(), w.v.clone().pin_memory()
    out_h = torch.zeros(w.q.shape, dtype=torch.bfloat16).pin_memory()
    ops.paged_attn_decode_append(q_h, k_h, v_h, d["k_cache"], d["v_cache"], d["context_lens"], d["block_tables"], w.scale, out=out_h)
    torch.cuda.synchronize()
    d2 = to_dev(w)
    want = ops.paged_attn_decode_append(d2["q"], d2["k"], d2["v"], d2["k_cache"], d2["v_cache"], d2["context_lens"],
                                        d2["block_tables"], w.scale)
    torch.cuda.synchronize()
    assert torch.equal(out_h, want.cpu())
    assert torch.equal(d["k_cache"].view(torch.int16), d2["k_cache"].view(torch.int16))
    assert torch.equal(d["v_cache"].view(torch.int16), d2["v_cache"].view(torch.int16))


@pytest.mark.parametrize("hq,hkv", [(24, 8), (40, 8), (7, 1), (48, 8), (8, 8)])
def test_fused_append_decode_any_group_size(hq, hkv):
    """The one-launch step for query-head groups of 3, 5, 7, 6 and 1 heads (Qwen3-14B is 40 over 8)."""
    rng = np.random.default_rng(hq + 1)
    lens = rng.integers(100, 2600, size=10)
    w = workloads._decode_workload("any-group", 78 + hq, hq, hkv, lens, workloads._pool_size(lens), "cpu")
    got, want = _fused_step(w)
    assert_close(got, want, ATOL_BF16, RTOL_BF16, f"fused step {hq}q/{hkv}kv")


def test_fused_append_decode_long_context_full_size():
    """The long-context shape at full size (batch 256, contexts up to 32768 tokens, half the batch sharing the
    pages of a 2048-token prefix) through the one-launch step: pools bit for bit on the GPU against the inputs,
    outputs of the shortest, a middle and the longest sequence against the oracle."""
    w = workloads.config4(device="cuda", longest_at_cap=True)
    cl, bt = w.context_lens_tensor().cuda(), w.block_tables_tensor().cuda()
    got = ops.paged_attn_decode_append(w.q, w.k, w.v, w.k_cache, w.v_cache, cl, bt, w.scale)
    torch.cuda.synchronize()
    at = w.slot_mapping.cuda().long()
    assert torch.equal(w.k_cache.view(-1, w.n_kv_heads, 128)[at], w.k) and torch.equal(w.v_cache.view(-1, w.n_kv_heads, 128)[at], w.v)
    order = np.argsort(w.context_lens)
    for b in (int(order[0]), int(order[len(order) // 2]), int(order[-1])):
        pages = torch.tensor(w.block_tables[b], device="cuda")
        kc, vc = w.k_cache[pages].cpu(), w.v_cache[pages].cpu()
        local = torch.arange(len(pages), dtype=torch.int32)[None]
        want = oracle.paged_decode(w.q[b:b + 1].cpu(), kc, vc, torch.tensor([w.context_lens[b]], dtype=torch.int32), local, w.scale)
        assert_close(got[b:b + 1], want, ATOL_BF16, RTOL_BF16, f"fused step, long-context, sequence {b} ({w.context_lens[b]} tokens)")
