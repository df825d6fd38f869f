"""Small-K parity matrix for the CTA-pair tensor-core GEMM (the kernel that runs the large FP8 x FP8 and
BF16 x BF16 problems, both operands K-contiguous).  It is only selected for problems with at least as many
256 x 256 tiles as there are SM pairs, so its cases are large in m and n; K stays small so that the oracle
remains cheap.  Every case asserts which kernel the library actually launched (e5b_last_route), so a later
change of the selection rule cannot silently empty this matrix.

Covered against the oracle, every output and every padding byte (the reference's criterion,
tests/test_util.h:82-89,145-147, over a case matrix in the style of tests/test_gemm.cu:13-46): ragged m / n
(zero-filled TMA tails and the element-wise epilogue), the 1 / 2 / 4-slice last round, short K where the
stage ring never wraps and K that is not a multiple of the 128-byte stage, all FP8 pairings and BF16 x BF16,
all five output dtypes, tight and padded leading dimensions, row- and column-wise scales, bias of three
dtypes, beta with C = D and with a C tensor of another dtype; plus the exact one-MAC model on a pair-sized
problem, bit for bit.
"""
import numpy as np
import pytest

import oracle as orc
from harness import BF16, E4M3, E5M2, FP16, FP32, GemmCase, GemmData, check_tolerance, from_dev, to_dev

pytestmark = pytest.mark.gpu

SMS = 148                     # B200
SHAPES = [(2304, 2304),       # 81 tiles: 7 left for the last round -> cut into 4 slices
          (2560, 2816),       # 110 tiles: 36 left -> 2 slices
          (4864, 3840),       # 285 tiles: 63 left -> whole tiles
          (2321, 2309)]       # ragged in both directions (100 tiles, 26 left -> 2 slices)
KS = [16, 144, 784, 1040]
PAIRINGS = [(E5M2, E5M2), (E5M2, E4M3), (E4M3, E4M3), (E4M3, E5M2), (BF16, BF16)]
OUTS = [BF16, FP32, FP16, E5M2, E4M3]


def takes_pair_kernel(c):
    """The library's selection rule for the CTA-pair kernels, restated: TN storage, an unmixed FP8 or BF16 pair,
    m and n of at least 512 and at least one 256 x 256 tile per SM pair."""
    unmixed = (c.at in (E5M2, E4M3)) == (c.bt in (E5M2, E4M3)) and FP32 not in (c.at, c.bt)
    tiles = -(-c.m // 256) * -(-c.n // 256)
    return c.ta == 1 and c.tb == 0 and unmixed and c.m >= 512 and c.n >= 512 and tiles >= SMS // 2


def pair_cases():
    cases, idx = [], 0
    for si, (m, n) in enumerate(SHAPES):
        for k in KS:
            if m * n * k > 15e9:           # keeps the oracle to seconds: the biggest shape skips the longest K
                continue
            for rep in range(3):
                at, bt = PAIRINGS[idx % 5]
                dt = OUTS[(idx // 2 + si) % 5]
                mode = idx % 4             # 0, 3: beta = 0; 1: accumulate into D; 2: C tensor of another dtype
                ct = -1 if mode != 2 else OUTS[(idx + 3) % 5]
                beta = {0: 0.0, 1: 1.0, 2: 0.5, 3: 0.0}[mode]
                bias = [-1, BF16, FP32, E4M3][(idx // 3) % 4]
                vec = idx % 4 if at != BF16 else 0
                cases.append(GemmCase(1, 0, m, n, k, at, bt, dt, ct, bias, [1.0, 1.25, -0.5][idx % 3], beta, vec=vec,
                                      seed=500 + idx, tight=bool((idx // 2) % 2)))
                idx += 1
    return cases


CASES = pair_cases()


def test_every_case_meets_the_selection_rule():
    assert len(CASES) >= 40
    assert all(takes_pair_kernel(c) for c in CASES)
    # the matrix really spans what it claims to
    assert {c.dt for c in CASES} == set(OUTS) and {(c.at, c.bt) for c in CASES} == set(PAIRINGS)
    assert {c.tight for c in CASES} == {True, False} and {c.vec for c in CASES} == {0, 1, 2, 3}
    assert {c.bias for c in CASES} == {-1, BF16, FP32, E4M3}


def _run(case, **options):
    from e5m2effma_b200 import capi
    for name, v in options.items():
        capi.set_option(name, v)
    try:
        d = GemmData(case)
        got, amax = d.run_gpu()
        route = capi.last_route()
    finally:
        for name in options:
            capi.set_option(name, None)
    check_tolerance(d, got, amax)
    assert capi.gemm_fault() == 0
    return route


@pytest.mark.parametrize("case", CASES, ids=lambda c: c.label())
def test_pair_kernel_within_tolerance(case):
    """Library defaults: the problem must land on one of the CTA-pair kernels."""
    from e5m2effma_b200 import capi
    route = _run(case)
    assert route in (capi.ROUTE_TC_PAIR, capi.ROUTE_TC_PAIR_WIDE), f"launched route {route}, not a CTA-pair kernel"


@pytest.mark.parametrize("case", CASES[::3], ids=lambda c: c.label())
def test_pair_kernel_256_tiles_within_tolerance(case):
    """The 256 x 256 double-buffered pair kernel specifically (wide tiles switched off)."""
    from e5m2effma_b200 import capi
    assert _run(case, TC_WIDE=0) == capi.ROUTE_TC_PAIR


@pytest.mark.parametrize("case", CASES[1::7], ids=lambda c: c.label())
def test_same_data_without_tail_slices_and_on_single_ctas(case):
    """The same problems with the last round left whole, and on the one-CTA kernel: all within the same bound."""
    from e5m2effma_b200 import capi
    assert _run(case, TC_SPLIT=0) in (capi.ROUTE_TC_PAIR, capi.ROUTE_TC_PAIR_WIDE)
    assert _run(case, TC_PAIR=0) in (capi.ROUTE_TC_256, capi.ROUTE_TC_128)


WIDE_EXTRA = [GemmCase(1, 0, 3584, 3584, 272, E5M2, E4M3, E5M2, -1, BF16, 1.0, 0.0, vec=1, seed=901, tight=True),   # W = 512: 98 tiles, 24 left -> 2 slices
              GemmCase(1, 0, 4864, 3840, 144, E4M3, E4M3, BF16, -1, -1, 1.25, 1.0, vec=2, seed=902),                  # W = 512: 150 tiles, 2 left -> 2 slices
              GemmCase(1, 0, 8192, 512, 400, E5M2, E5M2, FP32, BF16, FP32, 1.0, 0.5, vec=3, seed=903, tight=True),    # a column shard: n = 512
              GemmCase(1, 0, 2500, 2100, 528, BF16, BF16, FP16, -1, -1, 1.0, 0.0, seed=904)]


@pytest.mark.parametrize("width", [512, 480, 384, 224])
@pytest.mark.parametrize("case", CASES[::4] + WIDE_EXTRA, ids=lambda c: c.label())
def test_wide_tiles_within_tolerance(case, width):
    """The wide-tile pair kernel at forced tile widths: full-width accumulators (512), a width whose half is not a
    multiple of the epilogue's 32-row step (480), widths with sliced last rounds, narrow tiles for column shards."""
    from e5m2effma_b200 import capi
    assert _run(case, TC_WIDE=width) == capi.ROUTE_TC_PAIR_WIDE


def test_pair_kernel_is_deterministic():
    from e5m2effma_b200 import capi
    d = GemmData(GemmCase(1, 0, 2321, 2309, 784, E5M2, E4M3, BF16, -1, BF16, 1.0, 0.0, vec=1, seed=77))
    a, am_a = d.run_gpu()
    assert capi.last_route() in (capi.ROUTE_TC_PAIR, capi.ROUTE_TC_PAIR_WIDE)
    b, am_b = d.run_gpu()
    assert np.array_equal(a, b) and am_a == am_b


@pytest.mark.parametrize("wide", [0, None], ids=["256-tiles", "default"])
@pytest.mark.parametrize("fa,fb", [(1, 1), (1, 0), (0, 0)], ids=["e5m2xe5m2", "e5m2xe4m3", "e4m3xe4m3"])
def test_pair_kernel_reproduces_the_one_mac_model(fa, fb, wide):
    """RN_BF16(acc + a*b) of the reference's exact model (tests/e5m2effma_ref.h:70-129) on a 2304 x 2304 x 16
    problem with one non-zero k: row i holds code i mod 256, column j code j mod 256, C a BF16 accumulator."""
    import torch
    from e5m2effma_b200 import capi
    rng = np.random.default_rng(10 * fa + fb)
    m = n = 2304
    k = 16
    ta, tb = (capi.E5M2 if fa else capi.E4M3), (capi.E5M2 if fb else capi.E4M3)

    def codes(count, e5m2):
        c = (np.arange(count) % 256).astype(np.uint8)
        ok = ((c & 0x7C) != 0x7C) if e5m2 else ((c & 0x7F) != 0x7F)
        return np.where(ok, c, 0x3C if e5m2 else 0x38).astype(np.uint8)     # non-finite codes -> 1.0

    ca, cb = codes(m, fa), codes(n, fb)
    A, B = np.zeros(m * k, np.uint8), np.zeros(n * k, np.uint8)
    A[np.arange(m) * k + 9] = ca
    B[np.arange(n) * k + 9] = cb
    C = rng.integers(0, 2 ** 16, m * n).astype(np.uint16)
    C = np.where((C & 0x7F80) == 0x7F80, C ^ 0x4000, C).astype(np.uint16)
    C = np.where(C == 0x8000, 0, C).astype(np.uint16)     # (-0) + (-0): the only case where a GEMM and the model differ
    bA, pA = to_dev(A)
    bB, pB = to_dev(B)
    bD, pD = to_dev(C)
    capi.set_option("TC_WIDE", wide)
    try:
        st = capi.gemm(capi.OP_T, capi.OP_N, m, n, k, 1.0, capi.tensor(pA, ta), k, capi.tensor(pB, tb), k, 1.0, None, 0,
                       capi.tensor(pD, capi.BF16), m, None, torch.cuda.current_stream().cuda_stream)
        route = capi.last_route()
    finally:
        capi.set_option("TC_WIDE", None)
    torch.cuda.synchronize()
    assert st == capi.OK, capi.last_error()
    assert route in (capi.ROUTE_TC_PAIR, capi.ROUTE_TC_PAIR_WIDE) and capi.gemm_fault() == 0
    got = from_dev(bD, np.uint16, m * n)
    jj, ii = np.meshgrid(np.arange(n), np.arange(m), indexing="ij")
    exp = orc.lane_n(ca[ii.ravel()], cb[jj.ravel()], C, fa, fb).astype(np.uint16)
    bad = np.flatnonzero(got != exp)
    assert bad.size == 0, f"{bad.size} of {m * n} outputs differ from the one-MAC model; first at {bad[0]}"
