"""Pins the CPU oracle: against golden vectors recorded from the reference's own host code
(tests/golden, made by tests/golden/make_golden.py) and, where the libraries compiled from the
reference sources are present (oracle/_ref), against those directly on larger sweeps.  Also the
known-answer vector of the reference's binding test (binds/python/tests/test_e5m2effma.py:118-125)."""
import ctypes
import os

import numpy as np
import pytest

import oracle as orc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_ENC = os.path.join(ROOT, "oracle", "_ref", "librefenc.so")


def same_floats(a_bits, b_bits):
    """Bitwise equality, except that any NaN equals any NaN (payloads are not part of the contract)."""
    a, b = a_bits.view(np.float32), b_bits.view(np.float32)
    return bool(np.all((a_bits == b_bits) | (np.isnan(a) & np.isnan(b))))


def test_encoders_match_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "encoders.npz"))
    x = g["x_bits"].view(np.float32)
    assert np.array_equal(orc.encode(orc.E4M3, x), g["e4m3"])
    assert np.array_equal(orc.encode(orc.E5M2, x), g["e5m2"])
    assert np.array_equal(orc.encode(orc.BF16, x), g["bf16"])
    assert np.array_equal(orc.encode(orc.FP16, x), g["fp16"])
    assert np.array_equal(orc.encode(orc.E4M3, x, 0.5), g["e4m3_half"])
    assert np.array_equal(orc.encode(orc.E5M2, x, 0.5), g["e5m2_half"])


def test_decoders_match_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "decoders.npz"))
    for name, dt in (("e4m3", orc.E4M3), ("e5m2", orc.E5M2)):
        assert same_floats(orc.decode(dt, g["codes"]).view(np.uint32), g[name])
        assert same_floats(orc.decode(dt, g["codes"], 0.5).view(np.uint32), g[name + "_half"])
    assert same_floats(orc.decode(orc.BF16, g["h_bits"]).view(np.uint32), g["bf16"])
    assert same_floats(orc.decode(orc.FP16, g["h_bits"]).view(np.uint32), g["fp16"])


def _finite(codes, e5):
    return (codes & 0x7C) != 0x7C if e5 else (codes & 0x7F) != 0x7F


def test_one_mac_matches_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "lane.npz"))
    for fa in (0, 1):
        for fb in (0, 1):
            t = f"{fa}{fb}"
            a, b, acc, res = (g[f"{n}_{t}"].astype(np.uint32) for n in ("a", "b", "acc", "res"))
            got = orc.lane_n(a, b, acc, fa, fb)
            # the exact model is defined on finite operands and finite accumulators
            dom = _finite(a, fa) & _finite(b, fb) & ((acc & 0x7F80) != 0x7F80)
            assert dom.sum() > 30000
            assert np.array_equal(got[dom], res[dom])


def test_known_answer_vector():
    x = np.array([1.0, np.inf, -1e6, 3.0], np.float32)
    codes, amax = orc.cast(x, orc.FP32, orc.E5M2, amax=0.0)
    assert list(codes) == [0x3C, 0x7B, 0xFB, 0x42]
    assert np.isinf(amax)
    assert list(orc.encode(orc.E5M2, np.array([np.pi], np.float32))) == [0x42]
    assert list(orc.encode(orc.E4M3, np.array([np.pi], np.float32))) == [0x45]
    assert list(orc.encode(orc.BF16, np.array([np.pi], np.float32))) == [0x4049]


def test_amax_drops_nan_keeps_inf():
    x = np.array([np.nan, 2.0, -3.0], np.float32)
    _, amax = orc.cast(x, orc.FP32, orc.BF16, amax=0.5)
    assert amax == 3.0
    _, amax = orc.cast(np.array([np.nan, -np.inf], np.float32), orc.FP32, orc.BF16, amax=1.0)
    assert np.isinf(amax)
    # long arrays take the vectorised / multi-threaded loop: same rule there
    rng = np.random.default_rng(3)
    bits = rng.integers(0, 2 ** 16, (1 << 20) + 37).astype(np.uint16)
    for threads in (1, 3):
        orc.set_threads(threads)
        assert np.isinf(orc.cast(bits, orc.BF16, orc.E4M3, None, 0.5, amax=0.0)[1])
        finite = np.where((bits & 0x7F80) == 0x7F80, 0, bits).astype(np.uint16)
        _, amax = orc.cast(finite, orc.BF16, orc.FP32, amax=0.0)
        assert amax == np.abs(orc.decode(orc.BF16, finite)).max()
    orc.set_threads(min(orc.usable_cpus(), 64))


def test_gemm_one_mac_equals_lane():
    """A k=16 GEMM with one non-zero product and a BF16 C (beta = 1) is RN_BF16(acc + a*b): the
    whole oracle GEMM path reproduces the one-MAC model."""
    rng = np.random.default_rng(5)
    m, n, k = 64, 48, 16
    for fa, ta in ((1, orc.E5M2), (0, orc.E4M3)):
        for fb, tb in ((1, orc.E5M2), (0, orc.E4M3)):
            A = np.zeros(m * k, np.uint8)
            B = np.zeros(n * k, np.uint8)
            ca = rng.integers(0, 256, m).astype(np.uint8)
            cb = rng.integers(0, 256, n).astype(np.uint8)
            ca = np.where(_finite(ca, fa), ca, 0x3C).astype(np.uint8)
            cb = np.where(_finite(cb, fb), cb, 0x3C).astype(np.uint8)
            A[np.arange(m) * k + 3] = ca
            B[np.arange(n) * k + 3] = cb
            C = rng.integers(0, 2 ** 16, m * n).astype(np.uint16)
            C = np.where((C & 0x7F80) == 0x7F80, 0x3F80, C).astype(np.uint16)
            D = np.zeros(m * n, np.uint16)
            orc.gemm(1, 0, m, n, k, 1.0, A, ta, k, B, tb, k, 1.0, C, orc.BF16, m, D, orc.BF16, m)
            ii, jj = np.meshgrid(np.arange(m), np.arange(n))
            exp = orc.lane_n(ca[ii.ravel()], cb[jj.ravel()], C, fa, fb)
            assert np.array_equal(D.astype(np.uint32), exp)


needs_ref = pytest.mark.skipif(not os.path.exists(REF_ENC), reason="oracle/_ref not built (reference sources absent)")


@needs_ref
def test_live_against_reference_host_code():
    enc = ctypes.CDLL(REF_ENC)
    p, f = ctypes.c_void_p, ctypes.c_float
    enc.ref_hstore_n.argtypes = [ctypes.c_int, p, ctypes.c_size_t, p, f]
    enc.ref_lane_n.argtypes = [ctypes.c_size_t, p, p, p, ctypes.c_int, ctypes.c_int, p]
    rng = np.random.default_rng(77)
    x = rng.integers(0, 2 ** 32, 3_000_000, dtype=np.uint64).astype(np.uint32).view(np.float32)
    for dt, st in ((orc.E4M3, np.uint8), (orc.E5M2, np.uint8), (orc.BF16, np.uint16), (orc.FP16, np.uint16)):
        for qs in (1.0, 0.03125):
            exp = np.zeros(x.size, st)
            enc.ref_hstore_n(dt, exp.ctypes.data, x.size, x.ctypes.data, qs)
            assert np.array_equal(orc.encode(dt, x, qs), exp), (dt, qs)
    # every (a, b) pair of every pairing against a corpus of accumulators (tests/check_ref.py:71-74 style)
    a, b = (v.ravel().astype(np.uint32) for v in np.meshgrid(np.arange(256), np.arange(256)))
    for fa in (0, 1):
        for fb in (0, 1):
            dom = _finite(a, fa) & _finite(b, fb)
            for acc0 in (0x0000, 0x8000, 0x3F80, 0xBF80, 0x0001, 0x7F7F, 0x4049, 0x0080):
                acc = np.full(a.size, acc0, np.uint32)
                exp = np.zeros(a.size, np.uint32)
                enc.ref_lane_n(a.size, a.ctypes.data, b.ctypes.data, acc.ctypes.data, fa, fb, exp.ctypes.data)
                got = orc.lane_n(a, b, acc, fa, fb)
                assert np.array_equal(got[dom], exp[dom]), (fa, fb, hex(acc0))
