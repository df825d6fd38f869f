"""K split over CTA pairs in the one-CTA tensor-core GEMM (few tiles, long K -- the column shard of a weight-gradient
GEMM on eight GPUs): two CTAs add up one half of K each, the second hands its partial sums to the first through
distributed shared memory.  Forced on small cases with the TC_KSPLIT switch and checked against the oracle on every
output; one case large enough to take the split by itself."""
import numpy as np
import pytest

from harness import BF16, E4M3, E5M2, FP16, FP32, GemmCase, GemmData, check_tolerance

pytestmark = pytest.mark.gpu


def _cases():
    out, seed = [], 400
    # operand pairs x layouts x outputs; ragged m / n, k from 2 k-blocks up, beta, row- and column-wise scales, bias
    for at, bt in ((E5M2, BF16), (BF16, E4M3), (E5M2, E4M3), (E4M3, E4M3), (BF16, BF16)):
        for (ta, tb), (m, n, k), dt, beta, vec in (((1, 0), (256, 256, 2048), FP32, 1.0, 0), ((1, 0), (200, 300, 1040), BF16, 0.0, 3),
                                                    ((0, 0), (384, 130, 512), E5M2, 0.5, 1), ((0, 1), (129, 257, 272), FP16, 0.0, 2),
                                                    ((1, 1), (520, 600, 4112), FP32, 1.0, 3)):
            seed += 1
            out.append(GemmCase(ta, tb, m, n, k, at, bt, dt, -1, BF16 if seed % 2 else -1, 1.0 if seed % 3 else 0.75, beta, vec=vec, seed=seed))
    return out


@pytest.mark.parametrize("case", _cases(), ids=lambda c: c.label())
def test_forced_k_split_within_tolerance(case):
    from e5m2effma_b200 import capi
    capi.set_option("TC_KSPLIT", 1)
    capi.set_option("TC_PAIR", 0)
    try:
        d = GemmData(case)
        got, amax = d.run_gpu()
        route = capi.last_route()
        again, _ = d.run_gpu()
    finally:
        capi.set_option("TC_KSPLIT", None)
        capi.set_option("TC_PAIR", None)
    assert route in (capi.ROUTE_TC_256_KSPLIT, capi.ROUTE_TC_128_KSPLIT), route
    assert capi.gemm_fault() == 0
    check_tolerance(d, got, amax)
    assert np.array_equal(got.view(np.uint8), again.view(np.uint8)), "two runs of the same problem differ"


def test_k_split_is_taken_by_a_wgrad_shard_and_can_be_switched_off():
    """2048 x 512 x 4096 E5M2 x BF16 accumulated into FP32 (32 tiles of 64 k-blocks on 148 SMs): split by default."""
    from e5m2effma_b200 import capi
    d = GemmData(GemmCase(1, 0, 2048, 512, 4096, E5M2, BF16, FP32, -1, -1, 1.0, 1.0, seed=431, tight=True))
    got, amax = d.run_gpu()
    assert capi.last_route() == capi.ROUTE_TC_256_KSPLIT and capi.gemm_fault() == 0
    check_tolerance(d, got, amax)
    capi.set_option("TC_KSPLIT", 0)
    try:
        got0, amax0 = d.run_gpu()
        assert capi.last_route() in (capi.ROUTE_TC_256, capi.ROUTE_TC_128)
    finally:
        capi.set_option("TC_KSPLIT", None)
    check_tolerance(d, got0, amax0)


@pytest.mark.parametrize("case", [GemmCase(1, 0, 2048, 1280, 512, E5M2, BF16, FP32, -1, -1, 1.0, 1.0, seed=441, tight=True),
                                  GemmCase(1, 0, 2000, 1300, 272, E5M2, E4M3, BF16, -1, BF16, 1.25, 0.0, vec=3, seed=442),
                                  GemmCase(0, 0, 1300, 2100, 144, BF16, BF16, FP32, BF16, -1, 1.0, 0.5, seed=443),
                                  GemmCase(0, 1, 2560, 1100, 1040, BF16, E5M2, E5M2, -1, -1, 1.0, 0.0, vec=2, seed=444)], ids=lambda c: c.label())
def test_forced_k_split_of_the_last_round(case):
    """More tiles than SMs with a sparse last round: the persistent CTAs run as clusters of two and share those tiles."""
    from e5m2effma_b200 import capi
    capi.set_option("TC_KSPLIT", 1)
    capi.set_option("TC_PAIR", 0)
    try:
        d = GemmData(case)
        got, amax = d.run_gpu()
        route = capi.last_route()
        again, _ = d.run_gpu()
    finally:
        capi.set_option("TC_KSPLIT", None)
        capi.set_option("TC_PAIR", None)
    assert route in (capi.ROUTE_TC_256_KTAIL, capi.ROUTE_TC_128_KTAIL), route
    assert capi.gemm_fault() == 0
    check_tolerance(d, got, amax)
    assert np.array_equal(got.view(np.uint8), again.view(np.uint8)), "two runs of the same problem differ"
