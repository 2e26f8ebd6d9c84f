"""The FP8 write kernel divides a bf16 value x by an fp32 scale s as
    r = RN(1 / s);  q0 = RN(x r);  q = RN(q0 + RN(x - s q0) r)
instead of an IEEE division.  This test replays that sequence in exact arithmetic on the host and
compares it with the correctly rounded quotient for all 128 significands of x against a sample of
the 2^23 significands of s (exponents do not matter inside the kernel's guarded range).
INFER_B200_EXHAUSTIVE=1 runs all 2^23 (about two minutes)."""
import os
from fractions import Fraction

import numpy as np


def _rn32(fr):
    c = np.float32(float(fr))
    cands = (np.nextafter(c, np.float32(-np.inf)), c, np.nextafter(c, np.float32(np.inf)))
    return min((abs(Fraction(float(v)) - fr), int(v.view(np.uint32)) & 1, v) for v in cands)[2]


def _check(sig):
    s = (sig.astype(np.uint32) | np.uint32(0x3F800000)).view(np.float32)        # [1, 2)
    r = (np.float32(1.0) / s).astype(np.float32)
    s64, r64 = s.astype(np.float64), r.astype(np.float64)
    bad = 0
    for m in range(128):
        x = np.float32(1.0 + m / 128.0)
        want = (x / s).astype(np.float32)
        q0 = (np.float64(x) * r64).astype(np.float32)            # 8 x 24 bit product: exact in f64, one rounding
        q064 = q0.astype(np.float64)
        rem = (np.float64(x) - s64 * q064).astype(np.float32)    # exact in f64, then the fma's single rounding
        t = rem.astype(np.float64) * r64                         # 24 x 24 bit product: exact in f64
        sum64 = q064 + t                                         # may round in f64: recheck near fp32 ties below
        q = sum64.astype(np.float32)
        d = np.abs(sum64 - q.astype(np.float64))
        half = np.spacing(np.abs(q)).astype(np.float64) / 2
        for i in np.nonzero(np.abs(d - half) <= 8 * np.spacing(np.abs(sum64)))[0]:
            q[i] = _rn32(Fraction(float(q0[i])) + Fraction(float(rem[i])) * Fraction(float(r[i])))
        bad += int(np.count_nonzero(q != want))
    return bad


def test_reciprocal_fma_division_is_correctly_rounded():
    if os.environ.get("INFER_B200_EXHAUSTIVE") == "1":
        sig = np.arange(2 ** 23, dtype=np.uint32)
    else:
        rng = np.random.default_rng(5)
        edge = np.concatenate([np.arange(4096), 2 ** 23 - 1 - np.arange(4096), 2 ** 22 + np.arange(-2048, 2048)])
        sig = np.unique(np.concatenate([edge, rng.integers(0, 2 ** 23, 2 ** 17)])).astype(np.uint32)
    assert _check(sig) == 0
