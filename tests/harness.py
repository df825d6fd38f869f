"""Shared helpers of the parity tests: seeded inputs in the reference's style, device buffers via
torch, the GPU call through the C interface, the oracle call, and the comparison rules.

Case layout follows the reference's run_case (tests/test_util.h:80-160): padded leading
dimensions (lda/ldb = round16 + 16, ldd = m + 3, ldc = m + 1), D prefilled with 0xA5 and the whole
padded buffer compared, so that a stray write is caught; scales 0.37 / 1.9 / 0.75 / 0.03125."""
import os
from dataclasses import dataclass

import numpy as np

import oracle as orc

E4M3, BF16, FP16, FP32, E5M2 = 0, 1, 2, 3, 4
NAMES = {E4M3: "E4M3", BF16: "BF16", FP16: "FP16", FP32: "FP32", E5M2: "E5M2"}
ULP_EPS = {BF16: 2.0 ** -8, FP16: 2.0 ** -11, FP32: 2.0 ** -24, E5M2: 2.0 ** -3, E4M3: 2.0 ** -4}


def is_fp8(t):
    return t in (E4M3, E5M2)


def fill(dtype, count, span, rng):
    """Storage array of `count` elements: FP8 -> uniformly random finite codes (every exponent),
    other dtypes -> uniform values in (-span, span)."""
    if dtype == E4M3:
        c = rng.integers(0, 256, count).astype(np.uint8)
        return np.where((c & 0x7F) == 0x7F, c ^ 1, c).astype(np.uint8)
    if dtype == E5M2:
        c = rng.integers(0, 256, count).astype(np.uint8)
        return np.where((c & 0x7C) == 0x7C, c ^ 4, c).astype(np.uint8)
    v = (rng.random(count, dtype=np.float32) * 2 - 1) * np.float32(span)
    return orc.encode(dtype, v)


def to_dev(arr, offset_bytes=0):
    """numpy storage -> (torch uint8 CUDA tensor holding it, device address of element 0)."""
    import torch
    raw = np.ascontiguousarray(arr).view(np.uint8).reshape(-1)
    buf = torch.empty(raw.size + offset_bytes + 16, dtype=torch.uint8, device="cuda")
    buf[offset_bytes:offset_bytes + raw.size] = torch.from_numpy(raw.copy()).cuda()
    return buf, buf.data_ptr() + offset_bytes


def from_dev(buf, np_dtype, count, offset_bytes=0):
    n = count * np.dtype(np_dtype).itemsize
    return buf[offset_bytes:offset_bytes + n].cpu().numpy().view(np_dtype).copy()


def ordered(dtype, raw):
    """Storage codes -> integers ordered like the values (sign-magnitude formats; +0 == -0)."""
    if dtype == FP32:
        u = raw.view(np.uint32).astype(np.int64)
        mag, neg = u & 0x7FFFFFFF, (u >> 31) != 0
    elif dtype in (BF16, FP16):
        u = raw.astype(np.int64)
        mag, neg = u & 0x7FFF, (u >> 15) != 0
    else:
        u = raw.astype(np.int64)
        mag, neg = u & 0x7F, (u >> 7) != 0
    return np.where(neg, -mag, mag)


@dataclass
class GemmCase:
    ta: int
    tb: int
    m: int
    n: int
    k: int
    at: int
    bt: int
    dt: int
    ct: int          # C dtype, -1: accumulate into D (C = NULL)
    bias: int        # bias dtype, -1: none
    alpha: float
    beta: float
    vec: int = 0     # bit 0: row-wise scale of A, bit 1: column-wise scale of B
    seed: int = 1
    tight: bool = False   # leading dimensions without padding (lda = k ..., ldd = m)

    def label(self):
        return (f"{'T' if self.ta else 'N'}{'T' if self.tb else 'N'} m={self.m} n={self.n} k={self.k} "
                f"A={NAMES[self.at]} B={NAMES[self.bt]} D={NAMES[self.dt]} "
                f"C={'accum' if self.ct < 0 else NAMES[self.ct]} bias={'-' if self.bias < 0 else NAMES[self.bias]} "
                f"a={self.alpha} b={self.beta} vec={self.vec}")


class GemmData:
    """Host-side buffers of one case (built once, used by the GPU run and by the oracle)."""

    def __init__(self, c: GemmCase):
        rng = np.random.default_rng(c.seed * 7919 + c.m * 31 + c.n * 17 + c.k)
        self.c = c
        a_kc, b_kc = c.ta == 1, c.tb == 0
        pad = 0 if c.tight else 16
        self.lda = ((c.k if a_kc else c.m) + 15) // 16 * 16 + pad
        self.ldb = ((c.k if b_kc else c.n) + 15) // 16 * 16 + pad
        self.ldd = c.m if c.tight else c.m + 3
        self.ldc = (c.m if c.tight else c.m + 1) if c.ct >= 0 else self.ldd
        self.cdt = c.ct if c.ct >= 0 else c.dt
        self.A = fill(c.at, self.lda * (c.m if a_kc else c.k), 2.0, rng)
        self.B = fill(c.bt, self.ldb * (c.n if b_kc else c.k), 2.0, rng)
        self.C = fill(self.cdt, self.ldc * c.n, 4.0, rng)
        if c.ct < 0:
            self.D0 = fill(c.dt, self.ldd * c.n, 4.0, rng)
            self.C = self.D0.copy()
        else:
            self.D0 = np.full(self.ldd * c.n * orc.esize(c.dt), 0xA5, np.uint8).view(orc.NP_STORAGE[c.dt]).copy()
        self.bias = fill(c.bias, c.m, 8.0, rng) if c.bias >= 0 else None
        self.va = bool(c.vec & 1) and is_fp8(c.at)
        self.vb = bool(c.vec & 2) and is_fp8(c.bt)
        self.sa = (0.25 + rng.integers(0, 1024, c.m) / 512.0).astype(np.float32) if self.va else np.array([0.37], np.float32)
        self.sb = (0.25 + rng.integers(0, 1024, c.n) / 512.0).astype(np.float32) if self.vb else np.array([1.9], np.float32)
        self.csinv = np.array([0.75], np.float32)
        self.qs = np.array([0.03125], np.float32)
        self.uses_c = c.beta != 0.0

    def oracle_args(self):
        c = self.c
        return dict(transa=c.ta, transb=c.tb, m=c.m, n=c.n, k=c.k, alpha=c.alpha, A=self.A, a_dtype=c.at, lda=self.lda,
                    B=self.B, b_dtype=c.bt, ldb=self.ldb, beta=c.beta, C=self.C if self.uses_c else None,
                    c_dtype=self.cdt, ldc=self.ldc, bias=self.bias, bias_dtype=c.bias if c.bias >= 0 else FP32,
                    a_sinv=self.sa if is_fp8(c.at) else None, a_outer=self.va,
                    b_sinv=self.sb if is_fp8(c.bt) else None, b_outer=self.vb,
                    c_sinv=self.csinv if is_fp8(self.cdt) else None)

    def run_oracle(self, order=0):
        c = self.c
        D = self.D0.copy()
        amax = orc.gemm(D=D, d_dtype=c.dt, ldd=self.ldd, d_scale=self.qs if is_fp8(c.dt) else None, amax=0.0,
                        order=order, **self.oracle_args())
        return D, amax

    def run_wide(self):
        return orc.gemm_wide(**self.oracle_args())

    def run_gpu(self):
        import torch
        from e5m2effma_b200 import capi
        c = self.c
        keep = []

        def dev(arr):
            b, p = to_dev(arr)
            keep.append(b)
            return b, p

        _, pA = dev(self.A)
        _, pB = dev(self.B)
        _, pC = dev(self.C)
        bD, pD = dev(self.D0)
        _, psa = dev(self.sa)
        _, psb = dev(self.sb)
        _, pcs = dev(self.csinv)
        _, pqs = dev(self.qs)
        bam, pam = dev(np.zeros(1, np.float32))
        A = capi.tensor(pA, c.at, psa, None, None, 1 if self.va else 0)
        B = capi.tensor(pB, c.bt, psb, None, None, 1 if self.vb else 0)
        C = capi.tensor(pC, self.cdt, pcs)
        D = capi.tensor(pD, c.dt, pcs, pqs, pam)
        bias = None
        if self.bias is not None:
            _, pb = dev(self.bias)
            bias = capi.tensor(pb, c.bias)
        st = capi.gemm(c.ta, c.tb, c.m, c.n, c.k, c.alpha, A, self.lda, B, self.ldb, c.beta,
                       C if c.ct >= 0 else None, self.ldc, D, self.ldd, bias, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert st == capi.OK, (capi.status_string(st), capi.last_error())
        got = from_dev(bD, orc.NP_STORAGE[c.dt], self.ldd * c.n)
        amax = from_dev(bam, np.float32, 1)[0]
        return got, amax


def check_exact(data: GemmData, got, amax, order=0):
    exp, eamax = data.run_oracle(order)
    bad = int(np.count_nonzero(exp.view(np.uint8) != got.view(np.uint8)))
    if bad and data.c.dt == FP32:   # NaN payloads are not part of the contract
        e, g = exp.view(np.float32), got.view(np.float32)
        bad = int(np.count_nonzero(~((e.view(np.uint32) == g.view(np.uint32)) | (np.isnan(e) & np.isnan(g)))))
    assert bad == 0, f"{data.c.label()}: {bad} bytes differ from the ascending-k emulation"
    assert amax == eamax or (np.isnan(amax) and np.isnan(eamax)), f"{data.c.label()}: amax {amax} != {eamax}"


def check_tolerance(data: GemmData, got, amax):
    """|D - D_ref| <= 1 ulp of the output format + k * 2^-23 * sum|a*b|*|s| (accumulation order),
    evaluated in code space: the admissible value interval is encoded with the oracle's encoders
    and widened by one code on each side.  Padding rows must keep their canary / initial bytes."""
    c = data.c
    ref, mag, fix = data.run_wide()           # (n, m) float64 each
    order_bound = c.k * 2.0 ** -23 * mag
    slack = 2.0 ** -21 * (np.abs(ref) + fix + mag)   # the handful of FP32 roundings of the epilogue
    lo, hi = ref - order_bound - slack, ref + order_bound + slack
    qs = float(data.qs[0]) if is_fp8(c.dt) else 1.0
    f32max = float(np.finfo(np.float32).max)
    enc = lambda v: orc.encode(c.dt, np.clip(v, -f32max, f32max).astype(np.float32), qs)
    olo, ohi = ordered(c.dt, enc(lo)), ordered(c.dt, enc(hi))
    g2 = got.reshape(c.n, data.ldd)
    og = ordered(c.dt, g2[:, :c.m])
    ok = (og >= np.minimum(olo, ohi) - 1) & (og <= np.maximum(olo, ohi) + 1)
    assert ok.all(), (f"{c.label()}: {int((~ok).sum())} outputs outside tolerance; first at "
                      f"{np.argwhere(~ok)[0]}, got code {og[~ok][0]}, window [{olo[~ok][0]}, {ohi[~ok][0]}]")
    d0 = data.D0.reshape(c.n, data.ldd)
    assert np.array_equal(g2[:, c.m:].view(np.uint8), d0[:, c.m:].view(np.uint8)), f"{c.label()}: padding rows overwritten"
    finite = np.isfinite(ref)
    ea = float(np.abs(ref[finite]).max()) if finite.any() else 0.0
    ab = float((order_bound + slack)[finite].max()) if finite.any() else 0.0
    assert abs(float(amax) - ea) <= ab + 2.0 ** -22 * ea, f"{c.label()}: amax {amax} vs {ea} (+-{ab})"


def force_simt(on):
    from e5m2effma_b200 import capi
    capi.set_option("FORCE_SIMT", 1 if on else None)


def reference_gemm_cases():
    """The case matrix of the reference's tests/test_gemm.cu:13-46."""
    outs = [BF16, FP32, FP16, E5M2, E4M3]
    ops = [E5M2, E4M3, BF16, FP32]
    sizes = [(1, 9, 16), (37, 45, 48), (200, 300, 144), (257, 129, 256)]
    cases, idx = [], 0
    for ta in (0, 1):
        for tb in (0, 1):
            for at in ops:
                for bt in ops:
                    m, n, k = sizes[idx % 4]
                    ct = -1 if idx % 5 == 1 else (outs[(idx + 1) % 5] if idx % 5 == 2 else outs[idx % 5])
                    bias = -1 if idx % 3 == 0 else (BF16 if idx % 3 == 1 else FP32)
                    beta = 1.0 if idx % 5 == 1 else (0.5 if idx % 4 == 3 else 0.0)
                    cases.append(GemmCase(ta, tb, m, max(n, 9), k, at, bt, outs[idx % 5], ct, bias,
                                          1.25 if idx % 2 else 1.0, beta, seed=idx + 1))
                    idx += 1
    cases.append(GemmCase(1, 0, 1100, 1300, 512, E5M2, E5M2, BF16, -1, FP32, 1.0, 1.0, seed=101))
    cases.append(GemmCase(0, 0, 1029, 1500, 256, E5M2, BF16, FP32, -1, -1, 0.5, 1.0, seed=102))
    cases.append(GemmCase(0, 0, 768, 640, 512, E5M2, E4M3, BF16, -1, -1, 1.0, 0.0, seed=103))
    cases.append(GemmCase(1, 0, 512, 640, 768, E4M3, E5M2, FP32, -1, -1, 1.0, 1.0, seed=104))
    v = 1
    for ta in (0, 1):
        for tb in (0, 1):
            for dt in (BF16, FP32):
                cases.append(GemmCase(ta, tb, 257, 129, 256, E4M3 if v == 2 else E5M2, E4M3 if v == 1 else E5M2, dt,
                                      -1 if dt == BF16 else BF16, FP32 if dt == FP32 else -1, 1.25,
                                      0.0 if dt == BF16 else 0.5, vec=v, seed=110 + len(cases)))
                v = v % 3 + 1
    cases.append(GemmCase(1, 0, 1100, 1300, 512, E5M2, BF16, BF16, -1, -1, 1.0, 0.0, vec=3, seed=120))
    return cases


def reference_gemv_cases():
    """The case matrix of the reference's tests/test_gemv.cu:8-24."""
    outs = [BF16, FP32, FP16, E5M2, E4M3]
    ops = [E5M2, E4M3, BF16, FP32]
    gs = [(1, 16), (33, 272), (300, 1024), (1000, 4112)]
    cases, idx = [], 0
    for at in (E5M2, E4M3):
        for bt in ops:
            for n in range(1, 9):
                m, k = gs[(n + bt + at) % 4]
                c = GemmCase(1, 0, m, n, k, at, bt, outs[idx % 5], -1 if n == 3 else outs[idx % 5],
                             -1 if idx % 3 == 0 else BF16, 0.75 if idx % 2 else 1.0,
                             1.0 if n == 3 else (-1.5 if idx % 4 == 1 else 0.0), seed=200 + idx)
                cases.append(c)
                if n in (1, 4, 8):
                    cases.append(GemmCase(**{**c.__dict__, "vec": 1 + (n & 2) + (2 if is_fp8(bt) else 0)}))
                idx += 1
    return cases
