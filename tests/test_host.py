"""Host-side logic: workload generators, KV-head sharding, and the 2-rank gather of
per-shard outputs (gloo on CPU, the oracle standing in for the kernels)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from infer_b200 import workloads
from infer_b200.sharding import gather_heads, shard_bounds
from oracle import paged_kv_oracle as oracle


def test_config0_shapes_and_slots():
    w = workloads.config0()
    assert w.batch == 8 and w.n_q_heads == 16 and w.n_kv_heads == 8 and w.num_blocks == 64
    assert all(64 <= n <= 1024 for n in w.context_lens)
    used = [p for t in w.block_tables for p in t]
    assert len(used) == len(set(used)) and all(0 <= p < 64 for p in used)
    for t, n, s in zip(w.block_tables, w.context_lens, w.slot_mapping.tolist()):
        assert len(t) == -(-n // 256)
        assert s == t[(n - 1) // 256] * 256 + (n - 1) % 256
    assert w.kv_bytes() == sum(w.context_lens) * 8 * 128 * 2 * 2


def test_config1_is_deterministic_and_sized():
    a = workloads.config1(with_pool=False)
    b = workloads.config1(with_pool=False)
    assert a.context_lens == b.context_lens and a.block_tables == b.block_tables
    assert a.batch == 64 and all(512 <= n <= 8192 for n in a.context_lens)
    assert a.num_blocks >= sum(-(-n // 256) for n in a.context_lens)
    assert 1.0e9 < a.kv_bytes() < 1.4e9


def test_config4_shares_prefix_pages():
    w = workloads.config4(batch=32, cap=4096, with_pool=False)
    first = [tuple(t[:8]) for t in w.block_tables[:16]]
    assert len(set(first)) == 1                       # the same 8 physical pages
    assert all(tuple(t[:8]) != first[0] for t in w.block_tables[16:])
    for p in first[0]:
        assert w.ref_counts[p] == 16
    assert w.kv_bytes(unique=True) < w.kv_bytes(unique=False)


def test_config2_chunk_slots_follow_the_page_lists():
    w = workloads.config2(n_seqs=3, max_prefix=600, chunk=300)
    assert w.slot_mapping.numel() == 900
    at = 0
    for t, n in zip(w.block_tables, w.context_lens):
        for pos in range(n - 300, n):
            assert w.slot_mapping[at] == t[pos // 256] * 256 + pos % 256
            at += 1


def test_sharded_oracle_equals_full_oracle():
    w = workloads.config0()
    kc, vc = w.k_cache.clone(), w.v_cache.clone()
    oracle.store_kvcache(w.k, w.v, kc, vc, w.slot_mapping)
    full = oracle.paged_decode(w.q, kc, vc, w.context_lens_tensor(), w.block_tables_tensor(), w.scale)
    parts = []
    for r in range(4):
        s = w.shard(r, 4)
        skc, svc = s.k_cache.clone(), s.v_cache.clone()
        oracle.store_kvcache(s.k, s.v, skc, svc, s.slot_mapping)
        parts.append(oracle.paged_decode(s.q, skc, svc, s.context_lens_tensor(), s.block_tables_tensor(), s.scale))
        lo, hi = shard_bounds(w.n_q_heads, r, 4)
        assert hi - lo == s.n_q_heads
    assert torch.equal(torch.cat(parts, dim=1), full)


def _rank_main(rank, world, port, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w = workloads.config0()
        s = w.shard(rank, world)
        kc, vc = s.k_cache.clone(), s.v_cache.clone()
        oracle.store_kvcache(s.k, s.v, kc, vc, s.slot_mapping)
        local = oracle.paged_decode(s.q, kc, vc, s.context_lens_tensor(), s.block_tables_tensor(), s.scale)
        full = gather_heads(local)
        if rank == 0:
            kc, vc = w.k_cache.clone(), w.v_cache.clone()
            oracle.store_kvcache(w.k, w.v, kc, vc, w.slot_mapping)
            want = oracle.paged_decode(w.q, kc, vc, w.context_lens_tensor(), w.block_tables_tensor(), w.scale)
            result.put(bool(torch.equal(full, want)))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(180)
def test_two_rank_head_sharding_over_gloo():
    ctx = mp.get_context("spawn")
    result = ctx.Queue()
    with socket.socket() as sock:            # a port the kernel reports free right now
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, result)) for r in range(2)]
    for p in procs:
        p.start()
    ok = result.get(timeout=150)
    for p in procs:
        p.join(30)
        assert p.exitcode == 0
    assert ok


def test_step_staging_round_trip():
    from infer_b200.staging import StepStaging
    spec = {"slots": ((7,), torch.int32), "q": ((3, 4, 128), torch.bfloat16), "bt": ((3, 5), torch.int32)}
    st = StepStaging(spec, "cpu")
    st.host["slots"].copy_(torch.arange(7, dtype=torch.int32))
    st.host["q"].fill_(0.5)
    st.host["bt"].fill_(-1)
    st.upload()
    assert st.dev["slots"].tolist() == list(range(7))
    assert float(st.dev["q"].float().sum()) == 0.5 * 3 * 4 * 128
    assert bool((st.dev["bt"] == -1).all())
    assert st.dev["q"].data_ptr() % 256 == st._dev.data_ptr() % 256      # every view is 256-byte aligned
