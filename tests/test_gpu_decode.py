"""Paged decode attention through the C ABI against the CPU oracle (bf16 pools)."""
import numpy as np
import pytest
import torch

from gpu_util import ATOL_BF16, RTOL_BF16, assert_close, to_dev
from infer_b200 import ops, workloads
from oracle import paged_kv_oracle as oracle

pytestmark = pytest.mark.gpu

VARIANTS = [("2", "0"), ("2", "2"), ("2", "4"), ("2", "8"), ("1", "0")]   # (kernel, heads per tile)


def _step(w, monkeypatch, impl="0", hpc="0"):
    """append + decode on the GPU, the same two calls on the oracle."""
    monkeypatch.setenv("INFER_B200_DECODE_IMPL", impl)
    monkeypatch.setenv("INFER_B200_DECODE_HPC", hpc)
    d = to_dev(w)
    ops.store_kvcache(d["k"], d["v"], d["k_cache"], d["v_cache"], d["slot_mapping"])
    got = ops.paged_attn_decode(d["q"], d["k_cache"], d["v_cache"], d["context_lens"], d["block_tables"], w.scale)
    torch.cuda.synchronize()
    kc, vc = w.k_cache.clone(), w.v_cache.clone()
    oracle.store_kvcache(w.k, w.v, kc, vc, w.slot_mapping)
    want = oracle.paged_decode(w.q, kc, vc, w.context_lens_tensor(), w.block_tables_tensor(), w.scale)
    return got, want


@pytest.mark.parametrize("impl,hpc", VARIANTS)
def test_decode_config0(monkeypatch, impl, hpc):
    got, want = _step(workloads.config0(), monkeypatch, impl, hpc)
    assert_close(got, want, ATOL_BF16, RTOL_BF16, f"config0 impl={impl} hpc={hpc}")


@pytest.mark.parametrize("impl,hpc", VARIANTS)
def test_decode_qwen3_8b_shape_reduced(monkeypatch, impl, hpc):
    got, want = _step(workloads.config1(batch=12, lo=200, hi=3000), monkeypatch, impl, hpc)
    assert_close(got, want, ATOL_BF16, RTOL_BF16, f"config1/12 impl={impl} hpc={hpc}")


@pytest.mark.parametrize("impl,hpc", [("2", "0"), ("2", "8"), ("1", "0")])
def test_decode_group8_shared_prefix_reduced(monkeypatch, impl, hpc):
    w = workloads.config4(batch=16, cap=3000)
    got, want = _step(w, monkeypatch, impl, hpc)
    assert_close(got, want, ATOL_BF16, RTOL_BF16, f"config4/16 impl={impl} hpc={hpc}")


@pytest.mark.parametrize("world", [2, 4, 8])
def test_decode_head_shards_match_full(monkeypatch, world):
    """Each KV-head shard computed on its own equals the matching slice of the oracle."""
    w = workloads.config0()
    kc, vc = w.k_cache.clone(), w.v_cache.clone()
    oracle.store_kvcache(w.k, w.v, kc, vc, w.slot_mapping)
    want = oracle.paged_decode(w.q, kc, vc, w.context_lens_tensor(), w.block_tables_tensor(), w.scale)
    per = w.n_q_heads // world
    for r in (0, world - 1):
        got, _ = _step(w.shard(r, world), monkeypatch)
        assert_close(got, want[:, r * per:(r + 1) * per], ATOL_BF16, RTOL_BF16, f"shard {r}/{world}")


@pytest.mark.parametrize("impl,hpc", VARIANTS)
def test_decode_edge_lengths(monkeypatch, impl, hpc):
    """Lengths around tile and page boundaries, an empty row, -1 padding, stale pool bytes."""
    monkeypatch.setenv("INFER_B200_DECODE_IMPL", impl)
    monkeypatch.setenv("INFER_B200_DECODE_HPC", hpc)
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
    ops.paged_attn_decode(q.cuda(), kc.cuda(), vc.cuda(), cl.cuda(), bt.cuda(), 0.09, out=out)
    torch.cuda.synchronize()
    want = oracle.paged_decode(q, kc, vc, cl, bt, 0.09)
    live = cl > 0
    assert_close(out[live.cuda()], want[live], ATOL_BF16, RTOL_BF16, f"edges impl={impl} hpc={hpc}")
    assert bool((out[~live.cuda()] == 7.0).all()), "row with context_len == 0 was written"


def test_decode_golden_sdpa(golden, monkeypatch):
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


def test_decode_full_size_subset_against_oracle(monkeypatch):
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


def test_decode_in_cuda_graph(monkeypatch):
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


def test_decode_rejects_bad_arguments():
    kc = torch.zeros(2, 256, 8, 128, dtype=torch.bfloat16, device="cuda")
    q = torch.zeros(1, 24, 128, dtype=torch.bfloat16, device="cuda")       # 24 % 8 == 0 but group 3
    cl = torch.ones(1, dtype=torch.int32, device="cuda")
    bt = torch.zeros(1, 1, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="geometry"):
        ops.paged_attn_decode(q, kc, kc, cl, bt, 0.1)
    with pytest.raises(RuntimeError):
        ops.paged_attn_decode(q[:, :16].contiguous(), kc, kc, cl.long(), bt, 0.1)
