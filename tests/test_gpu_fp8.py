"""FP8-e4m3 KV: append bit-exact (bytes and scales) against the oracle's rule, decode within
the FP8 tolerance."""
import pytest
import torch

from gpu_util import ATOL_FP8, RTOL_FP8, assert_close, bits_equal
from infer_b200 import ops, workloads
from infer_b200.metadata import chunk_slots
from oracle import paged_kv_oracle as oracle

pytestmark = pytest.mark.gpu


def _empty_pools(num_blocks, hkv, device):
    mk = lambda: torch.zeros(num_blocks, 256, hkv, 128, dtype=torch.uint8, device=device)
    ms = lambda: torch.zeros(num_blocks, hkv, dtype=torch.float32, device=device)
    return mk(), mk(), ms(), ms()


def _fill_both(w, rounds):
    """Builds the FP8 pools by appending every sequence's existing tokens in several calls
    (so pages see their scale grow between calls), on the GPU and on the oracle."""
    cpu = _empty_pools(w.num_blocks, w.n_kv_heads, "cpu")
    gpu = _empty_pools(w.num_blocks, w.n_kv_heads, "cuda")
    bounds = [0.0, 0.3, 0.35, 1.0][:rounds + 1] if rounds == 3 else [0.0, 1.0]
    for lo_f, hi_f in zip(bounds[:-1], bounds[1:]):
        slots = []
        for t, n in zip(w.block_tables, w.context_lens):
            slots.extend(chunk_slots(t, int(lo_f * (n - 1)), int(hi_f * (n - 1)), 256))
        if not slots:
            continue
        idx = torch.tensor(slots, dtype=torch.int64)
        k = w.k_cache.view(-1, w.n_kv_heads, 128)[idx]
        v = w.v_cache.view(-1, w.n_kv_heads, 128)[idx]
        s32 = idx.to(torch.int32)
        oracle.store_kvcache_fp8(k, v, *cpu, s32)
        ops.store_kvcache(k.cuda(), v.cuda(), gpu[0], gpu[1], s32.cuda(), gpu[2], gpu[3])
    return cpu, gpu


@pytest.mark.parametrize("rounds", [1, 3])
def test_fp8_append_bit_exact(rounds):
    w = workloads.config3()
    cpu, gpu = _fill_both(w, rounds)
    torch.cuda.synchronize()
    assert torch.equal(cpu[2], gpu[2].cpu()), "k scales differ"
    assert torch.equal(cpu[3], gpu[3].cpu()), "v scales differ"
    assert bits_equal(cpu[0], gpu[0]), "k bytes differ"
    assert bits_equal(cpu[1], gpu[1]), "v bytes differ"


@pytest.mark.parametrize("hkv,n_tokens", [(1, 5), (3, 37), (2, 8), (8, 1001)])
def test_fp8_append_odd_heads_skips_and_strided_rows(hkv, n_tokens):
    """Head counts that do not fill a warp's head pair, token counts off the 8-token strip,
    skipped rows (-1) inside a strip, slots in random order over few pages (many rows per page
    in one call), rows that are column slices of a wider buffer; two calls so scales grow."""
    gen = torch.Generator().manual_seed(500 + hkv * 31 + n_tokens)
    nb = max(2, -(-2 * n_tokens // 200))
    cpu = _empty_pools(nb, hkv, "cpu")
    gpu = _empty_pools(nb, hkv, "cuda")
    all_slots = torch.randperm(nb * 256, generator=gen)[:2 * n_tokens]
    for call in range(2):
        slots = all_slots[call * n_tokens:(call + 1) * n_tokens].to(torch.int32)
        slots[torch.rand(n_tokens, generator=gen) < 0.15] = -1
        qkv = (torch.randn(n_tokens, 3 * hkv * 128 + 64, generator=gen) * (1 + 4 * call)).bfloat16()
        k = qkv[:, 64:64 + hkv * 128].view(n_tokens, hkv, 128)
        v = qkv[:, 64 + hkv * 128:64 + 2 * hkv * 128].view(n_tokens, hkv, 128)
        oracle.store_kvcache_fp8(k, v, *cpu, slots)
        qkv_d = qkv.cuda()
        ops.store_kvcache(qkv_d[:, 64:64 + hkv * 128].view(n_tokens, hkv, 128),
                          qkv_d[:, 64 + hkv * 128:64 + 2 * hkv * 128].view(n_tokens, hkv, 128),
                          gpu[0], gpu[1], slots.cuda(), gpu[2], gpu[3])
    torch.cuda.synchronize()
    assert torch.equal(cpu[2], gpu[2].cpu()) and torch.equal(cpu[3], gpu[3].cpu()), "scales differ"
    assert bits_equal(cpu[0], gpu[0]) and bits_equal(cpu[1], gpu[1]), "bytes differ"


def test_fp8_append_extreme_magnitudes():
    """Rows whose scale lies outside the range of the kernel's short division sequence (tiny,
    subnormal and huge amplitudes), all-zero rows, and quotients that fall on e4m3 rounding ties."""
    gen = torch.Generator().manual_seed(77)
    hkv, nb = 2, 8
    cpu = _empty_pools(nb, hkv, "cpu")
    gpu = _empty_pools(nb, hkv, "cuda")
    amps = [2.0 ** -140, 2.0 ** -120, 2.0 ** -70, 2.0 ** -30, 1.0, 2.0 ** 40, 2.0 ** 70, 2.0 ** 110]
    for call in range(2):
        ks, vs, slots = [], [], []
        for page, amp in enumerate(amps):
            n = 40
            grid = torch.randint(-448, 449, (n, hkv, 128), generator=gen).float() / 2     # many exact ties
            grid[0] = 448.0 if call else 300.0                                            # pins amax; grows on call 2
            grid[5] = 0.0
            ks.append((grid * (amp / 448.0)).bfloat16())
            vs.append((torch.randn(n, hkv, 128, generator=gen) * amp).bfloat16())
            slots.extend(range(page * 256 + call * 100, page * 256 + call * 100 + n))
        k, v = torch.cat(ks), torch.cat(vs)
        s32 = torch.tensor(slots, dtype=torch.int32)
        oracle.store_kvcache_fp8(k, v, *cpu, s32)
        ops.store_kvcache(k.cuda(), v.cuda(), gpu[0], gpu[1], s32.cuda(), gpu[2], gpu[3])
    torch.cuda.synchronize()
    assert torch.equal(cpu[2], gpu[2].cpu()) and torch.equal(cpu[3], gpu[3].cpu()), "scales differ"
    assert bits_equal(cpu[0], gpu[0]) and bits_equal(cpu[1], gpu[1]), "bytes differ"


@pytest.mark.parametrize("impl", ["0", "1"], ids=["tma", "plain-loads"])
def test_fp8_decode_step(impl, monkeypatch):
    monkeypatch.setenv("INFER_B200_DECODE_IMPL", impl)
    w = workloads.config3()
    cpu, gpu = _fill_both(w, 3)
    # the decode step's own append, then attention
    oracle.store_kvcache_fp8(w.k, w.v, *cpu, w.slot_mapping)
    ops.store_kvcache(w.k.cuda(), w.v.cuda(), gpu[0], gpu[1], w.slot_mapping.cuda(), gpu[2], gpu[3])
    cl, bt = w.context_lens_tensor(), w.block_tables_tensor()
    got = ops.paged_attn_decode(w.q.cuda(), gpu[0], gpu[1], cl.cuda(), bt.cuda(), w.scale, k_scale=gpu[2], v_scale=gpu[3])
    torch.cuda.synchronize()
    assert bits_equal(cpu[0], gpu[0]) and torch.equal(cpu[2], gpu[2].cpu())
    want = oracle.paged_decode(w.q, cpu[0], cpu[1], cl, bt, w.scale, cpu[2], cpu[3])
    assert_close(got, want, ATOL_FP8, RTOL_FP8, "fp8 decode vs fp8 oracle")


@pytest.mark.parametrize("hkv", [2, 1, 3, 4], ids=["2-heads-per-tile", "1-head", "3-heads-odd", "4-heads-per-tile"])
@pytest.mark.parametrize("impl", ["0", "1"], ids=["tma", "plain-loads"])
def test_fp8_decode_group8_long_contexts(impl, hkv, monkeypatch):
    """8 query heads per KV head, contexts over several pages with different scales per page,
    lengths around the 16/32/64/128/256-token boundaries of the FP8 tiles; the KV head count
    decides how many heads share a tile (4, 2, or 1 when it is odd)."""
    monkeypatch.setenv("INFER_B200_DECODE_IMPL", impl)
    gen = torch.Generator().manual_seed(91)
    hq, nb = 8 * hkv, 40
    lens = [1, 17, 255, 256, 257, 600, 1300, 33, 64, 65, 129]
    cpu = _empty_pools(nb, hkv, "cpu")
    gpu = _empty_pools(nb, hkv, "cuda")
    perm = torch.randperm(nb, generator=gen).tolist()
    tables, at = [], 0
    for n in lens:
        need = -(-n // 256)
        pages = perm[at:at + need]
        at += need
        tables.append(pages + [-1] * (6 - need))
        # every page gets its own amplitude so that page scales differ a lot
        k = torch.randn(n, hkv, 128, generator=gen)
        v = torch.randn(n, hkv, 128, generator=gen)
        amp = torch.repeat_interleave(torch.rand(need, generator=gen) * 8 + 0.1, 256)[:n]
        k, v = (k * amp[:, None, None]).bfloat16(), (v * amp.flip(0)[:, None, None]).bfloat16()
        slots = torch.tensor(chunk_slots(pages, 0, n, 256), dtype=torch.int32)
        oracle.store_kvcache_fp8(k, v, *cpu, slots)
        ops.store_kvcache(k.cuda(), v.cuda(), gpu[0], gpu[1], slots.cuda(), gpu[2], gpu[3])
    q = torch.randn(len(lens), hq, 128, generator=gen).bfloat16()
    cl = torch.tensor(lens, dtype=torch.int32)
    bt = torch.tensor(tables, dtype=torch.int32)
    got = ops.paged_attn_decode(q.cuda(), gpu[0], gpu[1], cl.cuda(), bt.cuda(), 0.09, k_scale=gpu[2], v_scale=gpu[3])
    torch.cuda.synchronize()
    assert bits_equal(cpu[0], gpu[0]) and bits_equal(cpu[1], gpu[1])
    want = oracle.paged_decode(q, cpu[0], cpu[1], cl, bt, 0.09, cpu[2], cpu[3])
    assert_close(got, want, ATOL_FP8, RTOL_FP8, f"fp8 decode, group 8, impl {impl}")
