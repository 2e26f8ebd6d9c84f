"""Pools whose pages hold 512 tokens (the engine only requires block_size % 256 == 0,
infer/config.py:21) and the largest batch the decode kernels take (2048 sequences): append,
paged decode, chunked prefill and the FP8 variants against the oracle."""
import pytest
import torch

from gpu_util import ATOL_BF16, ATOL_FP8, RTOL_BF16, RTOL_FP8, assert_close, bits_equal
from infer_b200 import ops
from infer_b200.metadata import chunk_slots
from oracle import paged_kv_oracle as oracle

pytestmark = pytest.mark.gpu
BS = 512


def _layout(lens, nb, gen):
    perm = torch.randperm(nb, generator=gen).tolist()
    tables, at = [], 0
    for n in lens:
        need = -(-n // BS)
        tables.append(perm[at:at + need])
        at += need
    width = max(len(t) for t in tables)
    bt = torch.tensor([t + [-1] * (width - len(t)) for t in tables], dtype=torch.int32)
    return tables, bt


def test_bf16_append_decode_prefill_with_512_token_pages():
    gen = torch.Generator().manual_seed(512)
    hq, hkv, nb = 16, 4, 20
    prefixes, chunks = [0, 511, 700, 1300, 512], [300, 600, 1, 513, 40]
    lens = [p + c for p, c in zip(prefixes, chunks)]
    tables, bt = _layout(lens, nb, gen)
    kc = torch.randn(nb, BS, hkv, 128, generator=gen).bfloat16()
    vc = torch.randn(nb, BS, hkv, 128, generator=gen).bfloat16()
    tq = sum(chunks)
    q = torch.randn(tq, hq, 128, generator=gen).bfloat16()
    k = torch.randn(tq, hkv, 128, generator=gen).bfloat16()
    v = torch.randn(tq, hkv, 128, generator=gen).bfloat16()
    slots = torch.tensor([s for t, p, n in zip(tables, prefixes, lens) for s in chunk_slots(t, p, n, BS)], dtype=torch.int32)
    cu_q = torch.tensor([0] + list(torch.tensor(chunks).cumsum(0)), dtype=torch.int32)
    cu_k = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    dkc, dvc = kc.cuda(), vc.cuda()
    ops.store_kvcache(k.cuda(), v.cuda(), dkc, dvc, slots.cuda())
    got = ops.paged_attn_prefill(q.cuda(), dkc, dvc, cu_q.cuda(), cu_k.cuda(), max(chunks), max(lens), 0.09, bt.cuda())
    torch.cuda.synchronize()
    oracle.store_kvcache(k, v, kc, vc, slots)
    assert bits_equal(kc, dkc) and bits_equal(vc, dvc)
    want = oracle.paged_prefill(q, kc, vc, cu_q, cu_k, bt, 0.09)
    assert_close(got, want, ATOL_BF16, RTOL_BF16, "prefill, 512-token pages")
    cl = torch.tensor(lens, dtype=torch.int32)
    qd = torch.randn(len(lens), hq, 128, generator=gen).bfloat16()
    got = ops.paged_attn_decode(qd.cuda(), dkc, dvc, cl.cuda(), bt.cuda(), 0.09)
    assert_close(got, oracle.paged_decode(qd, kc, vc, cl, bt, 0.09), ATOL_BF16, RTOL_BF16, "decode, 512-token pages")


def test_fp8_bulk_and_stepwise_append_with_512_token_pages():
    """Runs of up to 512 rows: longer than the registers of the run kernel hold, so the tail of a run is
    read a second time; then single-row appends that raise scales; bytes and scales bit-exact."""
    gen = torch.Generator().manual_seed(513)
    hq, hkv, nb = 8, 2, 12
    lens = [1500, 513, 2047]
    tables, bt = _layout([n + 8 for n in lens], nb, gen)
    mk = lambda dev: (torch.zeros(nb, BS, hkv, 128, dtype=torch.uint8, device=dev), torch.zeros(nb, BS, hkv, 128, dtype=torch.uint8, device=dev),
                      torch.zeros(nb, hkv, device=dev), torch.zeros(nb, hkv, device=dev))
    cpu, gpu = mk("cpu"), mk("cuda")
    k = (torch.randn(sum(lens), hkv, 128, generator=gen) * torch.rand(sum(lens), 1, 1, generator=gen) * 4).bfloat16()
    v = torch.randn(sum(lens), hkv, 128, generator=gen).bfloat16()
    slots = torch.tensor([s for t, n in zip(tables, lens) for s in chunk_slots(t, 0, n, BS)], dtype=torch.int32)
    oracle.store_kvcache_fp8(k, v, *cpu, slots)
    ops.store_kvcache(k.cuda(), v.cuda(), gpu[0], gpu[1], slots.cuda(), gpu[2], gpu[3])
    cur = list(lens)
    for step in range(8):
        cur = [n + 1 for n in cur]
        ks = (torch.randn(len(lens), hkv, 128, generator=gen) * (1 + 3 * step)).bfloat16()
        vs = torch.randn(len(lens), hkv, 128, generator=gen).bfloat16()
        sl = torch.tensor([t[(n - 1) // BS] * BS + (n - 1) % BS for t, n in zip(tables, cur)], dtype=torch.int32)
        oracle.store_kvcache_fp8(ks, vs, *cpu, sl)
        ops.store_kvcache(ks.cuda(), vs.cuda(), gpu[0], gpu[1], sl.cuda(), gpu[2], gpu[3])
    torch.cuda.synchronize()
    assert torch.equal(cpu[2], gpu[2].cpu()) and torch.equal(cpu[3], gpu[3].cpu()), "scales differ"
    assert bits_equal(cpu[0], gpu[0]) and bits_equal(cpu[1], gpu[1]), "bytes differ"
    cl = torch.tensor(cur, dtype=torch.int32)
    q = torch.randn(len(lens), hq, 128, generator=gen).bfloat16()
    got = ops.paged_attn_decode(q.cuda(), gpu[0], gpu[1], cl.cuda(), bt.cuda(), 0.09, k_scale=gpu[2], v_scale=gpu[3])
    want = oracle.paged_decode(q, cpu[0], cpu[1], cl, bt, 0.09, cpu[2], cpu[3])
    assert_close(got, want, ATOL_FP8, RTOL_FP8, "fp8 decode, 512-token pages")


def test_decode_largest_batch():
    """2048 sequences (the limit of the tile-prefix table), lengths 0..300 with empty rows in between."""
    gen = torch.Generator().manual_seed(2048)
    b, hq, hkv = 2048, 8, 2
    lens = torch.randint(0, 301, (b,), generator=gen)
    lens[::97] = 0
    nb = int((lens + 255).div(256, rounding_mode="floor").sum()) + 1
    kc = torch.randn(nb, 256, hkv, 128, generator=gen).bfloat16()
    vc = torch.randn(nb, 256, hkv, 128, generator=gen).bfloat16()
    perm = torch.randperm(nb, generator=gen).tolist()
    rows, at = [], 0
    for n in lens.tolist():
        need = -(-n // 256)
        rows.append(perm[at:at + need] + [-1] * (2 - need))
        at += need
    bt = torch.tensor(rows, dtype=torch.int32)
    cl = lens.to(torch.int32)
    q = torch.randn(b, hq, 128, generator=gen).bfloat16()
    out = torch.full((b, hq, 128), 5.0, dtype=torch.bfloat16, device="cuda")
    ops.paged_attn_decode(q.cuda(), kc.cuda(), vc.cuda(), cl.cuda(), bt.cuda(), 0.09, out=out)
    torch.cuda.synchronize()
    want = oracle.paged_decode(q, kc, vc, cl, bt, 0.09)
    live = cl > 0
    assert_close(out[live.cuda()], want[live], ATOL_BF16, RTOL_BF16, "decode, batch 2048")
    assert bool((out[~live.cuda()] == 5.0).all())
    with pytest.raises(RuntimeError, match="geometry"):
        ops.paged_attn_decode(torch.zeros(2049, hq, 128, dtype=torch.bfloat16, device="cuda"), kc.cuda(), vc.cuda(),
                              torch.ones(2049, dtype=torch.int32, device="cuda"),
                              torch.zeros(2049, 2, dtype=torch.int32, device="cuda"), 0.09)
