"""Seeded random problems through e5ma_gemm: shapes around every tile and k-block boundary, all four storage
layouts, every operand pairing without FP32 (those run the ascending-k kernel and are covered bit for bit
elsewhere), every output dtype, padded and tight leading dimensions, row-wise scales, bias, beta with a C tensor
or accumulating into D.  Every output is checked against the oracle's tolerance bound, padding must stay
untouched, and no bounded wait may have run out."""
import numpy as np
import pytest

from harness import BF16, E4M3, E5M2, FP16, FP32, GemmCase, GemmData, check_tolerance

pytestmark = pytest.mark.gpu

EDGES_MN = [1, 7, 9, 31, 33, 63, 64, 65, 127, 128, 129, 191, 255, 256, 257, 300, 383, 385, 511, 513, 640, 777]
EDGES_K = [16, 32, 48, 64, 80, 112, 128, 144, 240, 256, 272, 496, 512, 528, 1040]


def fuzz_cases(count=160, seed=20241):
    rng = np.random.default_rng(seed)
    ops, outs = [E5M2, E4M3, BF16], [BF16, FP32, FP16, E5M2, E4M3]
    cases = []
    for idx in range(count):
        m, n = int(rng.choice(EDGES_MN)), int(rng.choice(EDGES_MN))
        if idx % 10 == 0:                     # now and then a problem with more tiles than SMs
            m, n = int(rng.integers(1500, 2600)), int(rng.integers(1500, 2600))
        k = int(rng.choice(EDGES_K))
        at, bt, dt = int(rng.choice(ops)), int(rng.choice(ops)), int(rng.choice(outs))
        mode = int(rng.integers(0, 3))        # 0: beta = 0, 1: accumulate into D, 2: separate C tensor
        ct = -1 if mode != 2 else int(rng.choice(outs))
        beta = 0.0 if mode == 0 else float(rng.choice([1.0, 0.5, -0.25]))
        bias = int(rng.choice([-1, -1, BF16, FP32, E4M3]))
        cases.append(GemmCase(int(rng.integers(0, 2)), int(rng.integers(0, 2)), m, n, k, at, bt, dt, ct, bias,
                              float(rng.choice([1.0, 1.25, -0.5])), beta, vec=int(rng.integers(0, 4)),
                              seed=1000 + idx, tight=bool(rng.integers(0, 2))))
    return cases


@pytest.mark.parametrize("case", fuzz_cases(), ids=lambda c: c.label())
def test_random_problem_within_tolerance(case):
    from e5m2effma_b200 import capi
    d = GemmData(case)
    got, amax = d.run_gpu()
    check_tolerance(d, got, amax)
    assert capi.gemm_fault() == 0
