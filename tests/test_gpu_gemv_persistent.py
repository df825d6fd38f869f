"""The persistent bulk-copy GEMV kernel (selected with the GEMV_KERNEL switch; the library's default is the
cp.async kernel, which measures faster) against the oracle, every output and every padding byte: both weight formats, X in BF16 / E5M2 / E4M3, batch 1..8,
k tails inside the last 1 KiB stage and inside a warp's 128-byte slice, ragged last row tiles, all output dtypes,
row-wise scales, bias, beta.  A BF16 X is multiplied on the FP16 tensor-core path when all of it converts to FP16
exactly and on the BF16 path otherwise; both are forced here through the data.  Case shapes follow the
reference's GEMV matrix (tests/test_gemv.cu:8-24), from one row tile to more tiles than SMs."""
import numpy as np
import pytest

import oracle as orc
from harness import BF16, E4M3, E5M2, FP16, FP32, GemmCase, GemmData, check_tolerance

pytestmark = pytest.mark.gpu
OUTS = [BF16, FP32, FP16, E5M2, E4M3]


def _run(case, x_mode=None, force=True):
    from e5m2effma_b200 import capi
    d = GemmData(case)
    if case.bt == BF16 and x_mode is not None:
        v = orc.decode(BF16, d.B, 1.0).astype(np.float32)
        if x_mode == "f16":          # multiples of 2^-8 below 4: every value is an FP16 number
            v = np.round(v * 256.0) / 256.0
        elif x_mode == "huge":       # beyond the FP16 range: the BF16 path must take over
            v = v * np.float32(2.0 ** 20)
        elif x_mode == "tiny":       # below FP16's subnormal grid
            v = v * np.float32(2.0 ** -30)
        d.B = orc.encode(BF16, v)
    if force:
        capi.set_option("GEMV_KERNEL", 2)
    try:
        got, amax = d.run_gpu()
        route = capi.last_route()
    finally:
        capi.set_option("GEMV_KERNEL", None)
    check_tolerance(d, got, amax)
    assert capi.gemm_fault() == 0
    assert route == capi.ROUTE_GEMV_PERSISTENT, f"route {route}"


def big_cases():
    cases, idx = [], 0
    for m, k in [(4741, 1024), (4736, 1040), (5000, 2192), (8192, 4096), (6000, 912)]:
        for at in (E5M2, E4M3):
            for bt in (BF16, E5M2, E4M3):
                n = 1 + idx % 8
                dt = OUTS[idx % 5]
                beta = [0.0, 1.0, -1.5][idx % 3]
                cases.append(GemmCase(1, 0, m, n, k, at, bt, dt, -1 if idx % 3 == 1 else dt, BF16 if idx % 2 else -1,
                                      0.75 if idx % 2 else 1.0, beta, vec=(idx % 2) + (2 if bt != BF16 and idx % 4 >= 2 else 0),
                                      seed=700 + idx, tight=bool(idx % 2)))
                idx += 1
    return cases


@pytest.mark.parametrize("case", big_cases(), ids=lambda c: c.label())
def test_persistent_gemv_within_tolerance(case):
    _run(case)


@pytest.mark.parametrize("x_mode", ["f16", "huge", "tiny"])
@pytest.mark.parametrize("n", [1, 5, 8])
def test_bf16_x_on_the_fp16_path_and_on_the_bf16_path(n, x_mode):
    _run(GemmCase(1, 0, 4800, n, 2064, E5M2, BF16, BF16, -1, -1, 1.0, 0.0, vec=1, seed=40 + n, tight=True), x_mode=x_mode)
    _run(GemmCase(1, 0, 4800, n, 1024, E4M3, BF16, FP32, -1, BF16, 1.25, 0.0, vec=0, seed=50 + n), x_mode=x_mode)


@pytest.mark.parametrize("m,k", [(1, 16), (33, 272), (300, 1024), (1000, 4112), (17, 8192)])
@pytest.mark.parametrize("bt", [BF16, E4M3])
def test_small_shapes_forced_onto_the_persistent_kernel(m, k, bt):
    for n in (1, 3, 8):
        _run(GemmCase(1, 0, m, n, k, E5M2, bt, BF16, -1, BF16, 1.0, 0.0, vec=1, seed=60 + n), force=True)


def test_persistent_gemv_is_deterministic():
    from e5m2effma_b200 import capi
    d = GemmData(GemmCase(1, 0, 8192, 8, 2048, E5M2, BF16, BF16, -1, -1, 1.0, 0.0, vec=1, seed=5, tight=True))
    capi.set_option("GEMV_KERNEL", 2)
    try:
        a, am_a = d.run_gpu()
        assert capi.last_route() == capi.ROUTE_GEMV_PERSISTENT
        b, am_b = d.run_gpu()
    finally:
        capi.set_option("GEMV_KERNEL", None)
    assert np.array_equal(a, b) and am_a == am_b
