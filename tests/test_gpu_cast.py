"""e5ma_cast on the GPU against the oracle, bit for bit: every dtype pair, random FP32 bit patterns
(NaN / Inf / subnormals included), every FP8 code, tails and unaligned pointers, scale and amax.
Shapes of the cases follow reference tests/test_e5m2effma.cu:147-185."""
import numpy as np
import pytest

import oracle as orc
from harness import BF16, E4M3, E5M2, FP16, FP32, from_dev, is_fp8, to_dev

pytestmark = pytest.mark.gpu
ALL = [E4M3, BF16, FP16, FP32, E5M2]


def gpu_cast(src, sdt, ddt, count, scale_inv=None, scale=None, amax0=0.0, src_off=0, dst_off=0):
    import torch
    from e5m2effma_b200 import capi
    bs, ps = to_dev(src, src_off)
    dst0 = np.full(count * orc.esize(ddt) + 32, 0xA5, np.uint8)
    bd, pd = to_dev(dst0, dst_off)
    keep = []
    def scalar(v):
        if v is None:
            return None
        b, p = to_dev(np.array([v], np.float32)); keep.append(b); return p
    bam, pam = to_dev(np.array([amax0], np.float32))
    S = capi.tensor(ps, sdt, scalar(scale_inv))
    D = capi.tensor(pd, ddt, None, scalar(scale), pam)
    st = capi.cast(S, D, count, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert st == capi.OK, capi.last_error()
    out = from_dev(bd, np.uint8, count * orc.esize(ddt) + 32, dst_off)
    assert (out[count * orc.esize(ddt):] == 0xA5).all(), "wrote past the end"
    return out[:count * orc.esize(ddt)].view(orc.NP_STORAGE[ddt]), from_dev(bam, np.float32, 1)[0]


def same(ddt, got, exp):
    if ddt == FP32:
        g, e = got.view(np.uint32), exp.view(np.uint32)
        return bool(np.all((g == e) | (np.isnan(got) & np.isnan(exp))))
    return np.array_equal(got, exp)


def source(sdt, n, rng):
    if sdt == FP32:
        x = rng.integers(0, 2 ** 32, n, dtype=np.uint64).astype(np.uint32).view(np.float32).copy()
        x[:256] = orc.decode(E4M3, np.arange(256, dtype=np.uint8))
        x[256:512] = orc.decode(E5M2, np.arange(256, dtype=np.uint8))
        return x
    if is_fp8(sdt):
        return rng.integers(0, 256, n).astype(np.uint8)
    return rng.integers(0, 2 ** 16, n).astype(np.uint16)


@pytest.mark.parametrize("sdt", ALL)
@pytest.mark.parametrize("ddt", ALL)
def test_cast_pair_bit_exact(sdt, ddt):
    rng = np.random.default_rng(100 * sdt + ddt)
    n = (1 << 20) + 37
    src = source(sdt, n, rng)
    si = 0.5 if is_fp8(sdt) else None
    sc = 0.5 if is_fp8(ddt) else None
    got, amax = gpu_cast(src, sdt, ddt, n, si, sc)
    exp, eamax = orc.cast(src, sdt, ddt, si, sc, amax=0.0)
    assert same(ddt, got, exp)
    assert amax == eamax or (np.isnan(amax) and np.isnan(eamax))


@pytest.mark.parametrize("ddt", [E5M2, E4M3, BF16, FP16])
def test_cast_fp32_random_bits_with_scale(ddt):
    rng = np.random.default_rng(ddt)
    n = 1 << 22
    x = source(FP32, n, rng)
    sc = 0.5 if is_fp8(ddt) else None
    got, _ = gpu_cast(x, FP32, ddt, n, None, sc)
    exp, _ = orc.cast(x, FP32, ddt, None, sc)
    assert np.array_equal(got, exp)


@pytest.mark.parametrize("t", [E5M2, E4M3])
def test_every_fp8_code_decodes_exactly(t):
    codes = np.arange(256, dtype=np.uint8)
    for ddt in (FP32, BF16, FP16):
        got, amax = gpu_cast(codes, t, ddt, 256, 0.5)
        exp, eamax = orc.cast(codes, t, ddt, 0.5, amax=0.0)
        assert same(ddt, got, exp)
        assert amax == eamax   # E5M2 has Inf codes: amax = inf; NaN codes are ignored


def test_known_answer_and_amax_reduction():
    x = np.array([1.0, np.inf, -1e6, 3.0], np.float32)
    got, amax = gpu_cast(x, FP32, E5M2, 4)
    assert list(got) == [0x3C, 0x7B, 0xFB, 0x42] and np.isinf(amax)
    got, amax = gpu_cast(np.array([0.5, -0.25, np.nan], np.float32), FP32, BF16, 3, amax0=2.0)
    assert amax == 2.0 and list(got) == [0x3F00, 0xBE80, 0x7FC0]


@pytest.mark.parametrize("src_off,dst_off", [(4, 0), (0, 2), (4, 6)])
def test_unaligned_pointers_take_the_scalar_path(src_off, dst_off):
    rng = np.random.default_rng(9)
    n = 70001
    x = source(FP32, n, rng)
    got, amax = gpu_cast(x, FP32, BF16, n, src_off=src_off, dst_off=dst_off)
    exp, eamax = orc.cast(x, FP32, BF16, amax=0.0)
    assert np.array_equal(got, exp) and (amax == eamax or np.isnan(eamax))


@pytest.mark.parametrize("n", [1, 15, 16, 17, 255, 4097])
def test_small_counts(n):
    rng = np.random.default_rng(n)
    x = (rng.standard_normal(n) * 100).astype(np.float32)
    got, amax = gpu_cast(x, FP32, E4M3, n, None, 2.0)
    exp, eamax = orc.cast(x, FP32, E4M3, None, 2.0, amax=0.0)
    assert np.array_equal(got, exp) and amax == eamax


@pytest.mark.parametrize("sdt,ddt", [(BF16, BF16), (E4M3, E5M2), (E5M2, E5M2), (BF16, FP16), (FP32, FP32)])
def test_in_place_cast_between_dtypes_of_one_size(sdt, ddt):
    """src == dst: the reference allows it (same-dtype casts act as copy + amax, src/e5m2effma.cu:85-101 checks no
    overlap); the result must be what the out-of-place cast gives."""
    import torch
    from e5m2effma_b200 import capi
    rng = np.random.default_rng(7 * sdt + ddt)
    n = (1 << 18) + 21
    src = source(sdt, n, rng)
    si = 0.5 if is_fp8(sdt) else None
    sc = 2.0 if is_fp8(ddt) else None
    exp, eamax = orc.cast(src, sdt, ddt, si, sc, amax=0.0)
    buf, p = to_dev(src)
    keep = [to_dev(np.array([v], np.float32)) for v in (si or 1.0, sc or 1.0, 0.0)]
    S = capi.tensor(p, sdt, keep[0][1])
    D = capi.tensor(p, ddt, None, keep[1][1], keep[2][1])
    st = capi.cast(S, D, n, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert st == capi.OK, capi.last_error()
    got = from_dev(buf, orc.NP_STORAGE[ddt], n)
    amax = from_dev(keep[2][0], np.float32, 1)[0]
    assert same(ddt, got, exp)
    assert amax == eamax or (np.isnan(amax) and np.isnan(eamax))
