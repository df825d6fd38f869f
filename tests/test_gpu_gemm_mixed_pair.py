"""Parity matrix for the CTA-pair kernel of mixed FP8 x BF16 problems (selected with the MIXED_PAIR switch; both
operands K-contiguous, enough 256 x 256 tiles for half of the SM pairs, k >= 512): FP8 on either side (an FP8 A runs the transposed epilogue),
both FP8 formats, K with and without a tail inside the last 64-element block and long enough for both rings to
wrap, ragged m / n, sliced last rounds, all output dtypes, accumulation into D and a separate C, row- / column-wise
scales, bias.  Every output and every padding byte against the oracle (the reference's criterion,
tests/test_util.h:82-89,145-147); each case asserts that this kernel really ran."""
import numpy as np
import pytest

from harness import BF16, E4M3, E5M2, FP16, FP32, GemmCase, GemmData, check_tolerance

pytestmark = pytest.mark.gpu
OUTS = [FP32, BF16, FP16, E5M2, E4M3]
SHAPES = [(2304, 2304), (2560, 2816), (2321, 2309), (4864, 1800)]
KS = [528, 1040, 2064]
PAIRINGS = [(E5M2, BF16), (BF16, E4M3), (E4M3, BF16), (BF16, E5M2)]


def cases():
    out, idx = [], 0
    for m, n in SHAPES:
        for k in KS:
            for rep in range(2):
                at, bt = PAIRINGS[idx % 4]
                dt = OUTS[idx % 5]
                mode = idx % 3                       # 0: beta = 0, 1: accumulate into D, 2: C of another dtype
                ct = -1 if mode != 2 else OUTS[(idx + 2) % 5]
                beta = [0.0, 1.0, 0.5][mode]
                vec = (1 if at != BF16 else 2) if idx % 2 else 0
                out.append(GemmCase(1, 0, m, n, k, at, bt, dt, ct, [-1, BF16, FP32][idx % 3], [1.0, 0.75][idx % 2], beta, vec=vec,
                                    seed=800 + idx, tight=bool((idx // 2) % 2)))
                idx += 1
    return out


CASES = cases()


@pytest.mark.parametrize("case", CASES, ids=lambda c: c.label())
def test_mixed_pair_kernel_within_tolerance(case):
    from e5m2effma_b200 import capi
    capi.set_option("MIXED_PAIR", 1)
    try:
        d = GemmData(case)
        got, amax = d.run_gpu()
        route = capi.last_route()
    finally:
        capi.set_option("MIXED_PAIR", None)
    check_tolerance(d, got, amax)
    assert capi.gemm_fault() == 0
    assert route == capi.ROUTE_TC_MIXED_PAIR, f"launched route {route}"


@pytest.mark.parametrize("case", CASES[::5], ids=lambda c: c.label())
def test_same_problems_on_the_one_cta_kernel(case):
    from e5m2effma_b200 import capi
    capi.set_option("MIXED_PAIR", 0)
    try:
        d = GemmData(case)
        got, amax = d.run_gpu()
        route = capi.last_route()
    finally:
        capi.set_option("MIXED_PAIR", None)
    check_tolerance(d, got, amax)
    one_cta = (capi.ROUTE_TC_256, capi.ROUTE_TC_128, capi.ROUTE_TC_256_KSPLIT, capi.ROUTE_TC_128_KSPLIT, capi.ROUTE_TC_256_KTAIL, capi.ROUTE_TC_128_KTAIL)
    assert route in one_cta and capi.gemm_fault() == 0


def test_mixed_pair_kernel_is_deterministic():
    from e5m2effma_b200 import capi
    d = GemmData(GemmCase(1, 0, 2321, 2309, 1040, E5M2, BF16, FP32, -1, -1, 1.0, 1.0, vec=1, seed=78))
    capi.set_option("MIXED_PAIR", 1)
    try:
        a, am_a = d.run_gpu()
        assert capi.last_route() == capi.ROUTE_TC_MIXED_PAIR
        b, am_b = d.run_gpu()
    finally:
        capi.set_option("MIXED_PAIR", None)
    assert np.array_equal(a.view(np.uint8), b.view(np.uint8)) and am_a == am_b
