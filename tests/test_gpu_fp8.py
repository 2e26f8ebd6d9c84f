"""FP8-e4m3 KV: append bit-exact (bytes and scales) against the oracle's rule, decode within
the FP8 tolerance."""
import pytest
import torch

from gpu_util import ATOL_FP8, RTOL_FP8, assert_close, bits_equal
from infer_b200 import ops, selftest, workloads
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


def _decode(hpc, *args, **kw):
    if hpc == 0:
        return ops.paged_attn_decode(*args, **kw)
    with selftest.variant(decode_heads_per_tile=hpc):
        return ops.paged_attn_decode(*args, **kw)


@pytest.mark.parametrize("hpc", [0, 1, 2, 8], ids=["default-4-heads", "1-head", "2-heads", "8-heads"])
def test_fp8_decode_step(hpc):
    w = workloads.config3()
    cpu, gpu = _fill_both(w, 3)
    # the decode step's own append, then attention
    oracle.store_kvcache_fp8(w.k, w.v, *cpu, w.slot_mapping)
    ops.store_kvcache(w.k.cuda(), w.v.cuda(), gpu[0], gpu[1], w.slot_mapping.cuda(), gpu[2], gpu[3])
    cl, bt = w.context_lens_tensor(), w.block_tables_tensor()
    got = _decode(hpc, w.q.cuda(), gpu[0], gpu[1], cl.cuda(), bt.cuda(), w.scale, k_scale=gpu[2], v_scale=gpu[3])
    torch.cuda.synchronize()
    assert bits_equal(cpu[0], gpu[0]) and torch.equal(cpu[2], gpu[2].cpu())
    want = oracle.paged_decode(w.q, cpu[0], cpu[1], cl, bt, w.scale, cpu[2], cpu[3])
    assert_close(got, want, ATOL_FP8, RTOL_FP8, "fp8 decode vs fp8 oracle")


@pytest.mark.parametrize("hkv", [2, 1, 3, 4], ids=["2-heads-per-tile", "1-head", "3-heads-odd", "4-heads-per-tile"])
@pytest.mark.parametrize("group", [8, 5, 3])
def test_fp8_decode_long_contexts_any_group(group, hkv):
    """8, 5 or 3 query heads per KV head, contexts over several pages with different scales per
    page, lengths around the 16/32/64/128/256-token boundaries of the FP8 tiles; the KV head count
    decides how many heads share a tile (4, 2, or 1 when it is odd)."""
    gen = torch.Generator().manual_seed(91)
    hq, nb = group * hkv, 40
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
    assert_close(got, want, ATOL_FP8, RTOL_FP8, f"fp8 decode, group {group}, {hkv} kv heads")


def test_fp8_steps_scales_grow_under_later_reads():
    """Prefill a few sequences, then 300 decode-shape appends (one row per sequence and step) in
    which occasional outlier rows raise a page's scale, so that rows written many steps earlier are
    re-encoded and later decode passes read them through the new scale.  Pools and scales must stay
    bit-exact against the oracle stepped the same way, and every tenth step's attention output
    within the FP8 tolerance of the oracle's."""
    gen = torch.Generator().manual_seed(1234)
    hkv, hq, nb, steps = 4, 16, 24, 300
    start = [200, 255, 40, 511, 1]
    perm = torch.randperm(nb, generator=gen).tolist()
    cpu = _empty_pools(nb, hkv, "cpu")
    gpu = _empty_pools(nb, hkv, "cuda")
    tables, at = [], 0
    for n in start:
        need = -(-(n + steps) // 256)
        pages = perm[at:at + need]
        at += need
        tables.append(pages)
        k = torch.randn(n, hkv, 128, generator=gen).bfloat16()
        v = torch.randn(n, hkv, 128, generator=gen).bfloat16()
        slots = torch.tensor(chunk_slots(pages, 0, n, 256), dtype=torch.int32)
        oracle.store_kvcache_fp8(k, v, *cpu, slots)
        ops.store_kvcache(k.cuda(), v.cuda(), gpu[0], gpu[1], slots.cuda(), gpu[2], gpu[3])
    width = max(len(t) for t in tables)
    bt = torch.tensor([t + [-1] * (width - len(t)) for t in tables], dtype=torch.int32)
    bt_d = bt.cuda()
    lens = list(start)
    for step in range(steps):
        lens = [n + 1 for n in lens]
        k = torch.randn(len(start), hkv, 128, generator=gen)
        v = torch.randn(len(start), hkv, 128, generator=gen)
        if step % 7 == 3:                                   # an outlier row: this page's scale has to grow
            row = step % len(start)
            k[row] *= 6.0 + step / 20.0
            v[row, step % hkv] *= 9.0
        k, v = k.bfloat16(), v.bfloat16()
        slots = torch.tensor([t[(n - 1) // 256] * 256 + (n - 1) % 256 for t, n in zip(tables, lens)], dtype=torch.int32)
        oracle.store_kvcache_fp8(k, v, *cpu, slots)
        ops.store_kvcache(k.cuda(), v.cuda(), gpu[0], gpu[1], slots.cuda(), gpu[2], gpu[3])
        if step % 10 == 9 or step == steps - 1:
            q = torch.randn(len(start), hq, 128, generator=gen).bfloat16()
            cl = torch.tensor(lens, dtype=torch.int32)
            got = ops.paged_attn_decode(q.cuda(), gpu[0], gpu[1], cl.cuda(), bt_d, 0.09, k_scale=gpu[2], v_scale=gpu[3])
            torch.cuda.synchronize()
            assert torch.equal(cpu[2], gpu[2].cpu()) and torch.equal(cpu[3], gpu[3].cpu()), f"scales differ at step {step}"
            assert bits_equal(cpu[0], gpu[0]) and bits_equal(cpu[1], gpu[1]), f"bytes differ at step {step}"
            want = oracle.paged_decode(q, cpu[0], cpu[1], cl, bt, 0.09, cpu[2], cpu[3])
            assert_close(got, want, ATOL_FP8, RTOL_FP8, f"fp8 decode after step {step}")


def test_fp8_outlier_stress_qwen3_8b_shape_reduced():
    """The 1 %-outliers-times-20 stress of the FP8 configuration on the Qwen3-8B head layout
    (32q/8kv) with contexts of several pages: append bit-exact, decode within tolerance."""
    w = workloads.config1(batch=10, lo=300, hi=2600, seed=1013)
    gen = torch.Generator().manual_seed(1013)
    for t in (w.k, w.k_cache):
        spike = torch.rand(t.shape, generator=gen) < 0.01
        t[spike] = (t[spike].float() * 20).to(t.dtype)
    cpu, gpu = _fill_both(w, 3)
    oracle.store_kvcache_fp8(w.k, w.v, *cpu, w.slot_mapping)
    ops.store_kvcache(w.k.cuda(), w.v.cuda(), gpu[0], gpu[1], w.slot_mapping.cuda(), gpu[2], gpu[3])
    cl, bt = w.context_lens_tensor(), w.block_tables_tensor()
    got = ops.paged_attn_decode(w.q.cuda(), gpu[0], gpu[1], cl.cuda(), bt.cuda(), w.scale, k_scale=gpu[2], v_scale=gpu[3])
    torch.cuda.synchronize()
    assert torch.equal(cpu[2], gpu[2].cpu()) and torch.equal(cpu[3], gpu[3].cpu())
    assert bits_equal(cpu[0], gpu[0]) and bits_equal(cpu[1], gpu[1])
    want = oracle.paged_decode(w.q, cpu[0], cpu[1], cl, bt, w.scale, cpu[2], cpu[3])
    assert_close(got, want, ATOL_FP8, RTOL_FP8, "fp8 outlier stress, 32q/8kv")


@pytest.mark.parametrize("n_seqs,run_len", [(2048, 1), (1500, 3), (40, 40)])
def test_fp8_append_large_calls_in_short_runs(n_seqs, run_len):
    """Calls of more than 1024 tokens whose runs are short (the step of a large decode batch: one row per
    sequence, every sequence on pages of its own; a few rows each; 40-row runs) are routed to other kernels than
    a chunk's long runs: three calls on the same pages, magnitudes growing, so that scales grow and pages are
    re-encoded; bytes and scales bit-exact."""
    hkv = 2
    gen = torch.Generator().manual_seed(n_seqs * 7 + run_len)
    pages = torch.randperm(n_seqs, generator=gen)
    cpu = _empty_pools(n_seqs, hkv, "cpu")
    gpu = _empty_pools(n_seqs, hkv, "cuda")
    for step in range(3):
        first = 11 + step * run_len
        slots = (pages[:, None] * 256 + first + torch.arange(run_len)[None, :]).reshape(-1).to(torch.int32)
        k = (torch.randn(slots.numel(), hkv, 128, generator=gen) * (1.0 + step)).bfloat16()
        v = (torch.randn(slots.numel(), hkv, 128, generator=gen) * (3.0 - step)).bfloat16()
        oracle.store_kvcache_fp8(k, v, *cpu, slots)
        ops.store_kvcache(k.cuda(), v.cuda(), gpu[0], gpu[1], slots.cuda(), gpu[2], gpu[3])
    torch.cuda.synchronize()
    assert torch.equal(cpu[2], gpu[2].cpu()) and torch.equal(cpu[3], gpu[3].cpu()), "scales differ"
    assert bits_equal(cpu[0], gpu[0]) and bits_equal(cpu[1], gpu[1]), "bytes differ"
