"""Fused per-head RMSNorm + rotary embedding + KV append against the CPU restatement of the
reference's four separate steps.  V rows and untouched slots must be bit-exact.  q and the
rotated k follow the reference's rounding steps; the fp32 variance is summed in a different
order on the GPU, so a few values per hundred thousand start one bf16 unit apart before the
rotation, whose subtraction can turn that into a few units of a small result.  The checks:
at least 99.9 % of the elements bit-identical, the rest within the bf16 attention tolerance."""
from pathlib import Path

import numpy as np
import pytest
import torch

from gpu_util import bits_equal
from infer_b200 import ops
from infer_b200.metadata import chunk_slots
from oracle import paged_kv_oracle as oracle

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).resolve().parent / "golden"


def rope_cache(max_position, theta=1000000.0, d=128):
    inv_freq = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    freqs = torch.einsum("i,j -> ij", torch.arange(max_position, dtype=torch.float32), inv_freq)
    return torch.cat((freqs.cos(), freqs.sin()), dim=-1).bfloat16()


def check_near_bit_exact(got, want, what):
    from gpu_util import ATOL_BF16, RTOL_BF16, assert_close
    frac, worst = ulp_report(got, want)
    assert frac < 1e-3, (what, "fraction of differing elements", frac, "worst ulp distance", worst)
    assert_close(got, want, ATOL_BF16, RTOL_BF16, what)


def ulp_report(got, want):
    """Fraction of elements that differ and the largest difference in bf16 units in the last place."""
    g = got.cpu().view(torch.int16).to(torch.int32)
    w = want.view(torch.int16).to(torch.int32)
    # map sign-magnitude bf16 bit patterns to a monotone integer line
    key = lambda b: torch.where(b < 0, -(b & 0x7FFF), b)
    d = (key(g) - key(w)).abs()
    return float((d > 0).float().mean()), int(d.max())


def test_fused_golden_bits(golden):
    """On the golden case the q output equals, bit for bit, what the reference's RMSNorm and
    rotary functions produced."""
    g = golden["norm_rope"]
    gen = torch.Generator().manual_seed(g["seed"])
    t, h, d = g["t"], g["h"], 128
    x = (torch.randn(t, h, d, generator=gen) * 1.7).bfloat16()
    weight = (1.0 + 0.1 * torch.randn(d, generator=gen)).bfloat16()
    inv_freq = 1.0 / (g["theta"] ** (torch.arange(0, d, 2, dtype=torch.bfloat16) / d))
    freqs = torch.einsum("i,j -> ij", torch.arange(g["max_position"], dtype=torch.bfloat16), inv_freq)
    cache = torch.cat((freqs.cos(), freqs.sin()), dim=-1)
    positions = torch.tensor(g["positions"], dtype=torch.int64)
    kc = torch.zeros(2, 256, 1, 128, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    k = x[:, :1].contiguous()
    slots = torch.arange(t, dtype=torch.int32)
    q_out = ops.qk_norm_rope_append(x.cuda(), k.cuda(), k.cuda(), weight.cuda(), weight.cuda(), g["eps"], positions.cuda(),
                                    cache.cuda(), kc, vc, slots.cuda())
    torch.cuda.synchronize()
    want = torch.from_numpy(np.load(GOLD / "norm_rope_out.npy")).view(torch.bfloat16)
    check_near_bit_exact(q_out, want, "q vs the reference's functions")
    assert bits_equal(kc.view(-1, 128)[:t], q_out[:, 0])      # k went through the same arithmetic into its slots


@pytest.mark.parametrize("t,hq,hkv", [(64, 32, 8), (1, 16, 8), (700, 16, 8), (33, 2, 1), (5, 6, 3), (17, 40, 8), (9, 4, 1)])
def test_fused_matches_oracle(t, hq, hkv):
    gen = torch.Generator().manual_seed(t * 7 + hq)
    d, nb = 128, 8
    qkv = (torch.randn(t, (hq + 2 * hkv) * d, generator=gen) * 2).bfloat16()
    q = qkv[:, :hq * d].view(t, hq, d)
    k = qkv[:, hq * d:(hq + hkv) * d].view(t, hkv, d)
    v = qkv[:, (hq + hkv) * d:].view(t, hkv, d)
    qw = (1 + 0.2 * torch.randn(d, generator=gen)).bfloat16()
    kw = (1 + 0.2 * torch.randn(d, generator=gen)).bfloat16()
    cache = rope_cache(4096)
    positions = torch.randint(0, 4096, (t,), generator=gen, dtype=torch.int64)
    kc = torch.randn(nb, 256, hkv, d, generator=gen).bfloat16()
    vc = torch.randn(nb, 256, hkv, d, generator=gen).bfloat16()
    slots = torch.randperm(nb * 256, generator=gen)[:t].to(torch.int32)
    if t > 3:
        slots[3] = -1                                        # a padding row
    kc_g, vc_g = kc.cuda(), vc.cuda()
    qkv_g = qkv.cuda()
    q_out = ops.qk_norm_rope_append(qkv_g[:, :hq * d].view(t, hq, d), qkv_g[:, hq * d:(hq + hkv) * d].view(t, hkv, d),
                                    qkv_g[:, (hq + hkv) * d:].view(t, hkv, d), qw.cuda(), kw.cuda(), 1e-6, positions.cuda(),
                                    cache.cuda(), kc_g, vc_g, slots.cuda())
    torch.cuda.synchronize()
    want_q = oracle.qk_norm_rope_append(q, k, v, qw, kw, 1e-6, positions, cache, kc, vc, slots)
    assert bits_equal(vc_g, vc), "v pool must be bit-exact"
    check_near_bit_exact(q_out, want_q, "q")
    check_near_bit_exact(kc_g, kc, "k pool")
    untouched = torch.ones(nb * 256, dtype=torch.bool)
    untouched[slots[slots >= 0].long()] = False
    assert bits_equal(kc_g.view(-1, hkv, d)[untouched.cuda()], kc.view(-1, hkv, d)[untouched])


def test_fused_in_place_q_then_decode():
    """q rotated in place inside the fused qkv buffer, then a decode step on the appended
    pools, equals the oracle's norm + rope + store + paged decode."""
    from gpu_util import ATOL_BF16, RTOL_BF16, assert_close
    gen = torch.Generator().manual_seed(5)
    b, hq, hkv, d, nb = 6, 16, 8, 128, 12
    lens = [5, 256, 257, 300, 700, 64]
    perm = torch.randperm(nb, generator=gen).tolist()
    tables, at = [], 0
    for n in lens:
        need = -(-n // 256)
        tables.append(perm[at:at + need] + [-1] * (3 - need))
        at += need
    kc = torch.randn(nb, 256, hkv, d, generator=gen).bfloat16()
    vc = torch.randn(nb, 256, hkv, d, generator=gen).bfloat16()
    qkv = torch.randn(b, (hq + 2 * hkv) * d, generator=gen).bfloat16()
    qw = torch.ones(d).bfloat16()
    cache = rope_cache(2048)
    positions = torch.tensor([n - 1 for n in lens], dtype=torch.int64)
    slots = torch.tensor([t[(n - 1) // 256] * 256 + (n - 1) % 256 for t, n in zip(tables, lens)], dtype=torch.int32)
    kc_g, vc_g, qkv_g = kc.cuda(), vc.cuda(), qkv.cuda()
    qv = qkv_g[:, :hq * d].view(b, hq, d)
    ops.qk_norm_rope_append(qv, qkv_g[:, hq * d:(hq + hkv) * d].view(b, hkv, d), qkv_g[:, (hq + hkv) * d:].view(b, hkv, d),
                            qw.cuda(), qw.cuda(), 1e-6, positions.cuda(), cache.cuda(), kc_g, vc_g, slots.cuda(), q_out=qv)
    cl = torch.tensor(lens, dtype=torch.int32)
    bt = torch.tensor(tables, dtype=torch.int32)
    got = ops.paged_attn_decode(qv.contiguous(), kc_g, vc_g, cl.cuda(), bt.cuda(), d ** -0.5)
    torch.cuda.synchronize()
    q = qkv[:, :hq * d].view(b, hq, d)
    qn = oracle.qk_norm_rope_append(q, qkv[:, hq * d:(hq + hkv) * d].view(b, hkv, d), qkv[:, (hq + hkv) * d:].view(b, hkv, d),
                                    qw, qw, 1e-6, positions, cache, kc, vc, slots)
    want = oracle.paged_decode(qn, kc, vc, cl, bt, d ** -0.5)
    assert_close(got, want, ATOL_BF16, RTOL_BF16, "fused pre-attention step + decode")
