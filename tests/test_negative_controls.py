"""Negative controls (CPU only), in the spirit of the reference's E5MA_NEGATIVE_CONTROLS build
(tests/test_e5m2effma.cu:39-60): deliberately wrong encoders and deliberately damaged GEMM results must be
caught by the same corpus and the same checker the parity tests use, so a green parity run means something."""
import numpy as np
import pytest

import oracle as orc
from harness import BF16, E4M3, E5M2, FP32, GemmCase, GemmData, check_exact, check_tolerance


def corpus():
    """Random bit patterns plus every rounding boundary of the three narrow formats and NaNs."""
    rng = np.random.default_rng(5)
    bits = rng.integers(0, 2 ** 32, 400_000, dtype=np.uint64).astype(np.uint32)
    ties16 = (rng.integers(0, 1 << 16, 50_000, dtype=np.uint64).astype(np.uint32) << 16) | 0x8000
    parts = [bits.view(np.float32), ties16.view(np.float32), np.array([np.nan, -np.nan], np.float32)]
    for dt in (E5M2, E4M3):
        codes = np.arange(256, dtype=np.uint8)
        codes = codes[((codes & 0x7C) != 0x7C) if dt == E5M2 else ((codes & 0x7F) != 0x7F)]
        grid = np.sort(np.unique(np.abs(orc.decode(dt, codes)))).astype(np.float64)
        mid = ((grid[:-1] + grid[1:]) / 2).astype(np.float32)
        parts += [mid, -mid]
    return np.concatenate(parts).astype(np.float32)


def bf16_truncate(x):                       # no rounding at all
    return (x.view(np.uint32) >> 16).astype(np.uint16)


def bf16_rne_without_nan_rule(x):           # the carry of the rounding add turns some NaNs into Inf / other NaNs
    u = x.view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def fp8_ties_away(dtype, x):
    """Round half away from zero instead of half to even, inside the normal range."""
    mant, bias, top = (2, 15, 57344.0) if dtype == E5M2 else (3, 7, 448.0)
    out = orc.encode(dtype, x)
    a = np.abs(x)
    inside = np.isfinite(x) & (a < top) & (a >= 2.0 ** (1 - bias))
    b = a.view(np.uint32).astype(np.uint64) + (1 << (22 - mant))
    code = ((((b >> 23) - (127 - bias)) << mant) | ((b >> (23 - mant)) & ((1 << mant) - 1))).astype(np.uint64)
    sign = ((x.view(np.uint32) >> 24) & 0x80).astype(np.uint64)
    return np.where(inside, sign | code, out).astype(np.uint8)


def fp8_flush_subnormals(dtype, x):
    out = orc.encode(dtype, x).copy()
    emask = 0x7C if dtype == E5M2 else 0x78
    sub = (out & emask) == 0
    out[sub] &= 0x80
    return out


def test_corpus_separates_wrong_bf16_encoders_from_the_oracle():
    x = corpus()
    good = orc.encode(BF16, x)
    assert np.count_nonzero(bf16_truncate(x) != good) > 1000
    assert np.count_nonzero(bf16_rne_without_nan_rule(x) != good) >= 1     # only NaN inputs tell them apart
    finite = ~np.isnan(x)
    assert np.array_equal(bf16_rne_without_nan_rule(x)[finite], good[finite])   # ... which shows the control is sharp


@pytest.mark.parametrize("dtype", [E5M2, E4M3])
def test_corpus_separates_wrong_fp8_encoders_from_the_oracle(dtype):
    x = corpus()
    good = orc.encode(dtype, x)
    away = fp8_ties_away(dtype, x)
    diff = away != good
    assert diff.any()
    # the two can only differ where the value sits exactly on a tie between two codes
    back = orc.decode(dtype, good[diff]).astype(np.float64)
    other = orc.decode(dtype, away[diff]).astype(np.float64)
    assert np.allclose((back + other) / 2, x[diff].astype(np.float64), rtol=0, atol=0)
    assert np.count_nonzero(fp8_flush_subnormals(dtype, x) != good) > 100


def small_case():
    return GemmData(GemmCase(1, 0, 70, 45, 64, E5M2, E4M3, BF16, -1, FP32, 1.25, 0.0, vec=1, seed=9))


def test_checkers_accept_the_oracle_and_reject_damage():
    d = small_case()
    good, amax = d.run_oracle()
    check_exact(d, good, amax)
    check_tolerance(d, good, amax)

    # one output moved by a few codes
    bad = good.copy()
    bad.reshape(d.c.n, d.ldd)[7, 11] += np.uint16(8)
    with pytest.raises(AssertionError, match="differ"):
        check_exact(d, bad, amax)
    with pytest.raises(AssertionError, match="outside tolerance"):
        check_tolerance(d, bad, amax)

    # a padding element written
    bad = good.copy()
    bad.reshape(d.c.n, d.ldd)[3, d.c.m] ^= np.uint16(1)
    with pytest.raises(AssertionError):
        check_exact(d, bad, amax)
    with pytest.raises(AssertionError, match="padding"):
        check_tolerance(d, bad, amax)

    # a wrong amax
    with pytest.raises(AssertionError, match="amax"):
        check_exact(d, good, amax * 1.01)
    with pytest.raises(AssertionError, match="amax"):
        check_tolerance(d, good, amax * 1.01)


def test_tolerance_checker_rejects_a_dropped_k_block():
    """A kernel that skipped 16 of the 64 k values would pass a loose check; it must not pass this one."""
    d = small_case()
    good, amax = d.run_oracle()
    short = GemmData(d.c)
    short.A = d.A.copy().reshape(d.c.m, d.lda)
    short.A[:, 48:64] = 0                       # op(A) is K-contiguous here: zero the last 16 k of every row
    short.A = short.A.reshape(-1)
    damaged, damaged_amax = short.run_oracle()
    with pytest.raises(AssertionError):
        check_tolerance(d, damaged, damaged_amax)
