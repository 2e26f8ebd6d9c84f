"""KV append through the C ABI: cache contents bit-exact against the oracle."""
import pytest
import torch

from gpu_util import bits_equal, to_dev
from infer_b200 import ops, workloads
from oracle import paged_kv_oracle as oracle

pytestmark = pytest.mark.gpu


def _check(w):
    d = to_dev(w)
    ops.store_kvcache(d["k"], d["v"], d["k_cache"], d["v_cache"], d["slot_mapping"])
    kc, vc = w.k_cache.clone(), w.v_cache.clone()
    oracle.store_kvcache(w.k, w.v, kc, vc, w.slot_mapping)
    torch.cuda.synchronize()
    assert bits_equal(d["k_cache"], kc), "k pool differs"
    assert bits_equal(d["v_cache"], vc), "v pool differs"


def test_append_config0_bit_exact():
    _check(workloads.config0())


def test_append_decode_shape_reduced():
    _check(workloads.config1(batch=16, lo=300, hi=2000))


def test_append_chunked_prefill_shape_reduced():
    _check(workloads.config2(n_seqs=4, max_prefix=700, chunk=300))


def test_append_golden_strided_rows(golden):
    """Column slices of a fused qkv row, the reference's own call shape; digest of the whole
    pool equals the one its Triton kernel produced."""
    import hashlib
    g = golden["append"]
    gen = torch.Generator().manual_seed(g["seed"])
    n, hq, hkv, d = g["n"], g["hq"], g["hkv"], 128
    qkv = torch.randn(n, (hq + 2 * hkv) * d, generator=gen).bfloat16().cuda()
    key = qkv[:, hq * d:(hq + hkv) * d].view(n, hkv, d)
    value = qkv[:, (hq + hkv) * d:].view(n, hkv, d)
    kc = torch.zeros(g["num_blocks"], 256, hkv, d, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    ops.store_kvcache(key, value, kc, vc, torch.tensor(g["slots"], dtype=torch.int32, device="cuda"))
    dig = lambda t: hashlib.sha256(t.cpu().view(torch.uint8).numpy().tobytes()).hexdigest()
    assert dig(kc) == g["k_cache_digest"] and dig(vc) == g["v_cache_digest"]


def test_append_skips_negative_and_empty():
    kc = torch.zeros(2, 256, 8, 128, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    k = torch.randn(4, 8, 128, device="cuda").bfloat16()
    ops.store_kvcache(k, k, kc, vc, torch.tensor([3, -1, 511, -1], dtype=torch.int32, device="cuda"))
    ops.store_kvcache(k[:0], k[:0], kc, vc, torch.zeros(0, dtype=torch.int32, device="cuda"))
    torch.cuda.synchronize()
    flat = kc.view(-1, 8, 128)
    assert torch.equal(flat[3], k[0]) and torch.equal(flat[511], k[2])
    assert int((flat.abs().sum(dim=(1, 2)) > 0).sum()) == 2
    assert torch.equal(kc, vc)


def test_append_full_size_every_slot_written_once():
    """Config-2 scale (32768 rows): written slots hold their rows, all other slots keep
    their previous bytes."""
    n, hkv = 32768, 8
    num_blocks = 160
    gen = torch.Generator(device="cuda").manual_seed(11)
    k = torch.randn(n, hkv, 128, generator=gen, device="cuda").bfloat16()
    v = torch.randn(n, hkv, 128, generator=gen, device="cuda").bfloat16()
    kc = torch.randn(num_blocks, 256, hkv, 128, generator=gen, device="cuda").bfloat16()
    vc = torch.randn(num_blocks, 256, hkv, 128, generator=gen, device="cuda").bfloat16()
    k0, v0 = kc.clone(), vc.clone()
    slots = torch.randperm(num_blocks * 256, generator=gen, device="cuda")[:n].to(torch.int32)
    ops.store_kvcache(k, v, kc, vc, slots)
    torch.cuda.synchronize()
    idx = slots.long()
    assert torch.equal(kc.view(-1, hkv, 128)[idx], k) and torch.equal(vc.view(-1, hkv, 128)[idx], v)
    untouched = torch.ones(num_blocks * 256, dtype=torch.bool, device="cuda")
    untouched[idx] = False
    assert torch.equal(kc.view(-1, hkv, 128)[untouched], k0.view(-1, hkv, 128)[untouched])
    assert torch.equal(vc.view(-1, hkv, 128)[untouched], v0.view(-1, hkv, 128)[untouched])


def test_append_rejects_bad_arguments():
    kc = torch.zeros(1, 256, 8, 128, dtype=torch.bfloat16, device="cuda")
    k = torch.randn(2, 8, 128, device="cuda").bfloat16()
    with pytest.raises(RuntimeError):
        ops.store_kvcache(k, k, kc, kc, torch.zeros(2, dtype=torch.int64, device="cuda"))
    with pytest.raises(AssertionError):
        ops.store_kvcache(k, k, kc, kc, torch.zeros(3, dtype=torch.int32, device="cuda"))
    with pytest.raises(RuntimeError):
        ops.store_kvcache(k.float(), k.float(), kc, kc, torch.zeros(2, dtype=torch.int32, device="cuda"))
