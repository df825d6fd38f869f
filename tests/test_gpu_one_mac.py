"""The reference's exact one-MAC model, RN_BF16(acc + a*b) (tests/e5m2effma_ref.h:70-129, checked there by
tests/check_ref.py), swept through the WHOLE e5ma_gemm path on the GPU: a 256 x 256 x 16 problem whose row i of
op(A) holds code a = i in one k position and zeros elsewhere, column j of op(B) code b = j, C a BF16 accumulator
with beta = 1.  Every output is then RN_BF16(C[i,j] + a_i * b_j), so one launch covers all 65 536 code pairs of a
pairing for 65 536 accumulator values, and the result must equal the model bit for bit -- on the tensor cores too:
the product is exact and it is the only non-zero term of the sum."""
import numpy as np
import pytest

import oracle as orc
from harness import force_simt, from_dev, to_dev

pytestmark = pytest.mark.gpu


def finite(codes, e5m2):
    return ((codes & 0x7C) != 0x7C) if e5m2 else ((codes & 0x7F) != 0x7F)


def accumulators(rng, kind, count):
    if kind == "random":              # every exponent and sign, NaN / Inf excluded
        c = rng.integers(0, 2 ** 16, count).astype(np.uint16)
        return np.where((c & 0x7F80) == 0x7F80, c ^ 0x4000, c).astype(np.uint16)
    if kind == "zero":
        return np.zeros(count, np.uint16)
    if kind == "near":                # accumulators of the magnitude of the products: ties and cancellation
        return orc.encode(orc.BF16, (rng.standard_normal(count) * 4.0).astype(np.float32))
    return orc.encode(orc.BF16, (rng.standard_normal(count) * 1e-3).astype(np.float32))   # "tiny"


@pytest.mark.parametrize("simt", [False, True], ids=["tensor-core", "cuda-core"])
@pytest.mark.parametrize("kind", ["random", "zero", "near", "tiny"])
@pytest.mark.parametrize("fa,fb", [(1, 1), (1, 0), (0, 1), (0, 0)], ids=["e5m2xe5m2", "e5m2xe4m3", "e4m3xe5m2", "e4m3xe4m3"])
def test_gemm_reproduces_the_one_mac_model(fa, fb, kind, simt):
    import torch
    from e5m2effma_b200 import capi
    rng = np.random.default_rng(100 * fa + 10 * fb + len(kind))
    m = n = 256
    k = 16
    ta, tb = (capi.E5M2 if fa else capi.E4M3), (capi.E5M2 if fb else capi.E4M3)
    ca, cb = np.arange(256, dtype=np.uint8), np.arange(256, dtype=np.uint8)
    # codes with all exponent bits set are outside the operand contract (finite operands only): use 1.0 there
    one_a, one_b = (0x3C if fa else 0x38), (0x3C if fb else 0x38)
    ca = np.where(finite(ca, fa), ca, one_a).astype(np.uint8)
    cb = np.where(finite(cb, fb), cb, one_b).astype(np.uint8)
    A, B = np.zeros(m * k, np.uint8), np.zeros(n * k, np.uint8)
    A[np.arange(m) * k + 5] = ca
    B[np.arange(n) * k + 5] = cb
    C = accumulators(rng, kind, m * n)
    # a GEMM adds its 16 products to +0 before C is added, the one-MAC model adds the single product to C directly:
    # the two differ in one case only, (-0 product) + (-0 accumulator), so -0 accumulators are left out
    C = np.where(C == 0x8000, 0, C).astype(np.uint16)
    bA, pA = to_dev(A)
    bB, pB = to_dev(B)
    bD, pD = to_dev(C)                         # accumulate in place: D = RN(D + a*b)
    force_simt(simt)
    try:
        st = capi.gemm(capi.OP_T, capi.OP_N, m, n, k, 1.0, capi.tensor(pA, ta), k, capi.tensor(pB, tb), k, 1.0, None, 0,
                       capi.tensor(pD, capi.BF16), m, None, torch.cuda.current_stream().cuda_stream)
    finally:
        force_simt(False)
    torch.cuda.synchronize()
    assert st == capi.OK, capi.last_error()
    assert capi.gemm_fault() == 0
    got = from_dev(bD, np.uint16, m * n)
    jj, ii = np.meshgrid(np.arange(n), np.arange(m), indexing="ij")     # D is column-major: element (i, j) at i + j * m
    exp = orc.lane_n(ca[ii.ravel()], cb[jj.ravel()], C, fa, fb).astype(np.uint16)
    bad = np.flatnonzero(got != exp)
    assert bad.size == 0, (f"{bad.size} of 65536 differ; first: a={ca[ii.ravel()[bad[0]]]:#x} b={cb[jj.ravel()[bad[0]]]:#x} "
                           f"acc={C[bad[0]]:#06x} got={got[bad[0]]:#06x} want={exp[bad[0]]:#06x}")
