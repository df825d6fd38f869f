"""Seeded synthetic inputs for the configurations the library is measured on (the five in
BASELINE.json plus casts), generated on the GPU with torch and quantised with the library's own
e5ma_cast, following the quantisation recipe of the reference's Float8Tensor.from_float
(binds/python/e5m2effma/tensor.py:61-74): scale = max_fp8 / amax, codes = encode(x * scale),
scale_inv = 1 / scale.  Every workload exposes

    launch(stream)      one pass of the hot path through the C interface (device-resident inputs)
    units               algorithmic FLOPs (GEMM) or bytes (GEMV / AdamW / cast) of one pass
    host_inputs() / device_inputs / result   the buffers an end-to-end step has to move
"""
import torch


class _Codes:
    """dtype and enum codes of include/e5m2effma.h; kept here so that building a workload's input data does not
    load the library (the CPU reference arm of the benchmark generates the same inputs without it)."""
    E4M3, BF16, FP16, FP32, E5M2 = 0, 1, 2, 3, 4
    OP_N, OP_T = 0, 1
    OK = 0
    SCALING_OUTER = 1

    def __getattr__(self, name):          # everything else (calls, structures) comes from the real binding
        from . import capi as real
        return getattr(real, name)


capi = _Codes()

FP8_MAX = {capi.E5M2: 57344.0, capi.E4M3: 448.0}
TORCH_DT = {capi.E4M3: torch.float8_e4m3fn, capi.E5M2: torch.float8_e5m2, capi.BF16: torch.bfloat16,
            capi.FP16: torch.float16, capi.FP32: torch.float32}


def _check(st, what):
    if st != capi.OK:
        raise RuntimeError(f"{what}: {capi.status_string(st)}: {capi.last_error()}")


def _gen(seed, dev):
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    return g


QUANTIZER = None   # None: e5ma_cast on the GPU.  The reference arm of the benchmark installs a CPU encoder here.


def quantize(x32, dtype, scale=None):
    """FP32 tensor -> uint8 codes of `dtype` = encode(x * scale), via e5ma_cast (or the installed QUANTIZER)."""
    if QUANTIZER is not None:
        return QUANTIZER(x32, dtype, scale)
    out = torch.empty(x32.shape, dtype=torch.uint8, device=x32.device)
    s = None
    if scale is not None:
        s = torch.tensor([scale], dtype=torch.float32, device=x32.device)
    S = capi.tensor(x32.data_ptr(), capi.FP32)
    D = capi.tensor(out.data_ptr(), dtype, None, None if s is None else s.data_ptr())
    _check(capi.cast(S, D, x32.numel(), torch.cuda.current_stream().cuda_stream), "e5ma_cast")
    torch.cuda.current_stream().synchronize()
    return out


def randn_chunked(shape, std, seed, dev, out_dtype=torch.float32, chunk_rows=2048):
    """N(0, std) of a big 2-D shape without a full FP32 temporary when out_dtype is narrower."""
    g = _gen(seed, dev)
    out = torch.empty(shape, dtype=out_dtype, device=dev)
    for r0 in range(0, shape[0], chunk_rows):
        r1 = min(shape[0], r0 + chunk_rows)
        out[r0:r1] = (torch.randn((r1 - r0, shape[1]), generator=g, device=dev) * std).to(out_dtype)
    return out


class GemmWorkload:
    """e5ma_gemm, by default with both operands K-contiguous (the FP8 layout): A is [m, k] row-major storage
    (column-major k x m, transa = T), B is [n, k] (transb = N), D is [n, m] storage (column-major
    m x n, ldd = m).  transa = "N" stores A as [k, m] (lda = m), transb = "T" stores B as [k, n] (ldb = n): the
    same values, so the four layouts of one problem produce the same D."""

    kind = "gemm"

    def __init__(self, name, m, n, k, a_dtype, b_dtype, d_dtype, dev, a_std=1.0, b_std=1.0, a_uniform=None,
                 b_uniform=None, a_scaling="fixed", b_scaling="fixed", a_scale_inv=1.0, b_scale_inv=1.0, bias_std=None,
                 beta=0.0, d0_std=None, d_scale=None, want_amax=False, seed=0, transa="T", transb="N"):
        self.name, self.m, self.n, self.k = name, m, n, k
        self.transa, self.transb = transa, transb
        self.lda, self.ldb = (k if transa == "T" else m), (k if transb == "N" else n)
        self.a_dtype, self.b_dtype, self.d_dtype = a_dtype, b_dtype, d_dtype
        self.beta, self.dev = beta, dev
        self.A, self.sa, self.a_outer = self._operand((m, k), a_dtype, a_std, a_uniform, a_scaling, a_scale_inv, seed + 1)
        self.B, self.sb, self.b_outer = self._operand((n, k), b_dtype, b_std, b_uniform, b_scaling, b_scale_inv, seed + 2)
        if transa != "T":
            self.A = self.A.t().contiguous()
        if transb != "N":
            self.B = self.B.t().contiguous()
        self.bias = None
        if bias_std is not None:
            self.bias = (torch.randn(m, generator=_gen(seed + 3, dev), device=dev) * bias_std).to(torch.bfloat16)
        dt = TORCH_DT[d_dtype]
        if d0_std is not None:
            self.D = randn_chunked((n, m), d0_std, seed + 3, dev, dt)
        else:
            self.D = torch.zeros((n, m), dtype=torch.uint8 if d_dtype in FP8_MAX else dt, device=dev)
        self.D0 = self.D.clone() if beta != 0.0 else None
        self.d_scale = None if d_scale is None else torch.tensor([d_scale], dtype=torch.float32, device=dev)
        self.amax = torch.zeros(1, dtype=torch.float32, device=dev) if want_amax else None
        self.units = 2.0 * m * n * k
        self.unit_name = "FLOP"

    def _operand(self, shape, dtype, std, uniform, scaling, scale_inv, seed):
        dev = self.dev
        if dtype in (capi.BF16, capi.FP32):
            return randn_chunked(shape, std, seed, dev, TORCH_DT[dtype]), None, False
        if uniform is not None:
            x = (torch.rand(shape, generator=_gen(seed, dev), device=dev) * 2 - 1) * uniform
        else:
            x = randn_chunked(shape, std, seed, dev)
        if scaling == "fixed":          # codes = encode(x / scale_inv), scale_inv given
            codes = quantize(x, dtype, 1.0 / scale_inv)
            return codes, torch.tensor([scale_inv], dtype=torch.float32, device=dev), False
        if scaling == "tensor":         # scale_inv = amax / max_fp8
            amax = float(x.abs().max())
            codes = quantize(x, dtype, FP8_MAX[dtype] / amax)
            return codes, torch.tensor([amax / FP8_MAX[dtype]], dtype=torch.float32, device=dev), False
        amax = x.abs().amax(dim=1).clamp_min(1e-30)        # "outer": one factor per row
        x = x * (FP8_MAX[dtype] / amax)[:, None]
        codes = quantize(x, dtype)
        return codes, (amax / FP8_MAX[dtype]).to(torch.float32).contiguous(), True

    def tensors(self, A=None, B=None, D=None):
        A = self.A if A is None else A
        B = self.B if B is None else B
        D = self.D if D is None else D
        tA = capi.tensor(A.data_ptr(), self.a_dtype, None if self.sa is None else self.sa.data_ptr(), None, None,
                         capi.SCALING_OUTER if self.a_outer else 0)
        tB = capi.tensor(B.data_ptr(), self.b_dtype, None if self.sb is None else self.sb.data_ptr(), None, None,
                         capi.SCALING_OUTER if self.b_outer else 0)
        tD = capi.tensor(D.data_ptr(), self.d_dtype, None, None if self.d_scale is None else self.d_scale.data_ptr(),
                         None if self.amax is None else self.amax.data_ptr())
        tb = None if self.bias is None else capi.tensor(self.bias.data_ptr(), capi.BF16)
        return tA, tB, tD, tb

    def launch(self, stream, A=None, B=None, D=None):
        tA, tB, tD, tb = self.tensors(A, B, D)
        _check(capi.gemm(capi.OP_T if self.transa == "T" else capi.OP_N, capi.OP_N if self.transb == "N" else capi.OP_T,
                         self.m, self.n, self.k, 1.0, tA, self.lda, tB, self.ldb, self.beta, None, 0, tD, self.m, tb, stream), "e5ma_gemm")

    launches_per_pass = 1

    def io_tensors(self):
        """(inputs an end-to-end step uploads, result it reads back)"""
        ins = [self.A, self.B] + [t for t in (self.sa, self.sb, self.bias) if t is not None]
        if self.beta != 0.0:
            ins.append(self.D)
        return ins, [self.D] + ([self.amax] if self.amax is not None else [])


class AdamWorkload:
    kind = "adam"

    def __init__(self, name, count, dev, seed=0, with_copy=True):
        self.name, self.count, self.dev = name, count, dev
        chunk = 1 << 24
        self.p = torch.empty(count, dtype=torch.bfloat16, device=dev)
        self.g = torch.empty(count, dtype=torch.bfloat16, device=dev)
        gp, gg = _gen(seed + 1, dev), _gen(seed + 2, dev)
        for i in range(0, count, chunk):
            j = min(count, i + chunk)
            self.p[i:j] = (torch.randn(j - i, generator=gp, device=dev) * 0.02).to(torch.bfloat16)
            self.g[i:j] = (torch.randn(j - i, generator=gg, device=dev) * 1e-3).to(torch.bfloat16)
        self.m = torch.zeros(count, dtype=torch.bfloat16, device=dev)
        self.v = torch.zeros(count, dtype=torch.bfloat16, device=dev)
        self.q = torch.zeros(count, dtype=torch.uint8, device=dev) if with_copy else None
        self.qscale = torch.tensor([2048.0], dtype=torch.float32, device=dev)   # a power of two near 448 / amax
        self.amax = torch.zeros(1, dtype=torch.float32, device=dev)
        self.cfg = capi.AdamConfig(3e-4, 0.9, 0.999, 1e-8, 0.1, 1, 1, 1, 1.0)
        self.units = count * (15.0 if with_copy else 14.0)
        self.unit_name = "B"

    def launch(self, stream):
        P, G = capi.tensor(self.p.data_ptr(), capi.BF16), capi.tensor(self.g.data_ptr(), capi.BF16)
        M, V = capi.tensor(self.m.data_ptr(), capi.BF16), capi.tensor(self.v.data_ptr(), capi.BF16)
        Q = None if self.q is None else capi.tensor(self.q.data_ptr(), capi.E4M3, None, self.qscale.data_ptr(),
                                                    self.amax.data_ptr())
        _check(capi.adam(self.cfg, self.count, P, G, M, V, Q, stream), "e5ma_adam")

    def launch_range(self, stream, i0, i1):
        """The same step over elements [i0, i1) only (one rank's chunk of a sharded parameter set)."""
        P, G = capi.tensor(self.p.data_ptr() + 2 * i0, capi.BF16), capi.tensor(self.g.data_ptr() + 2 * i0, capi.BF16)
        M, V = capi.tensor(self.m.data_ptr() + 2 * i0, capi.BF16), capi.tensor(self.v.data_ptr() + 2 * i0, capi.BF16)
        Q = None if self.q is None else capi.tensor(self.q.data_ptr() + i0, capi.E4M3, None, self.qscale.data_ptr(),
                                                    self.amax.data_ptr())
        _check(capi.adam(self.cfg, i1 - i0, P, G, M, V, Q, stream), "e5ma_adam")

    launches_per_pass = 1

    def io_tensors(self):
        return [self.p, self.g, self.m, self.v], [self.p, self.m, self.v, self.q, self.amax]


class CastWorkload:
    kind = "cast"

    def __init__(self, name, count, src_dtype, dst_dtype, dev, seed=0):
        self.name, self.count, self.src_dtype, self.dst_dtype = name, count, src_dtype, dst_dtype
        es = {capi.FP32: 4, capi.BF16: 2, capi.FP16: 2, capi.E4M3: 1, capi.E5M2: 1}
        g = _gen(seed + 1, dev)
        if src_dtype in FP8_MAX:
            self.src = torch.randint(0, 120, (count,), generator=g, device=dev, dtype=torch.uint8)
        else:
            self.src = torch.empty(count, dtype=TORCH_DT[src_dtype], device=dev)
            for i in range(0, count, 1 << 24):
                j = min(count, i + (1 << 24))
                self.src[i:j] = torch.randn(j - i, generator=g, device=dev).to(TORCH_DT[src_dtype])
        self.dst = torch.zeros(count * es[dst_dtype], dtype=torch.uint8, device=dev)
        self.scale = torch.tensor([16.0], dtype=torch.float32, device=dev)
        self.amax = torch.zeros(1, dtype=torch.float32, device=dev)
        self.units = float(count) * (es[src_dtype] + es[dst_dtype])
        self.unit_name = "B"

    def launch(self, stream):
        S = capi.tensor(self.src.data_ptr(), self.src_dtype, self.scale.data_ptr())
        D = capi.tensor(self.dst.data_ptr(), self.dst_dtype, None, self.scale.data_ptr(), self.amax.data_ptr())
        _check(capi.cast(S, D, self.count, stream), "e5ma_cast")

    def launch_range(self, stream, i0, i1):
        es = {capi.FP32: 4, capi.BF16: 2, capi.FP16: 2, capi.E4M3: 1, capi.E5M2: 1}
        S = capi.tensor(self.src.data_ptr() + i0 * es[self.src_dtype], self.src_dtype, self.scale.data_ptr())
        D = capi.tensor(self.dst.data_ptr() + i0 * es[self.dst_dtype], self.dst_dtype, None, self.scale.data_ptr(), self.amax.data_ptr())
        _check(capi.cast(S, D, i1 - i0, stream), "e5ma_cast")

    launches_per_pass = 1

    def io_tensors(self):
        return [self.src], [self.dst, self.amax]


def make(name, dev, shrink=1):
    """Workloads by name.  shrink > 1 divides the sizes (tests and profiler captures)."""
    s = shrink
    if name == "c1":      # GEMM 4096^3 E5M2 x E5M2 -> BF16, values 8 * N(0,1), scale_inv 0.125 each
        return GemmWorkload("c1", 4096 // s, 4096 // s, 4096 // s, capi.E5M2, capi.E5M2, capi.BF16, dev, a_std=8.0, b_std=8.0,
                            a_scale_inv=0.125, b_scale_inv=0.125, seed=1000)
    if name in ("c2", "c2_bf16"):   # HYBRID dgrad: E5M2 gradient (row-wise) x E4M3 weights + BF16 bias -> E5M2 + amax
        first = name == "c2_bf16"   # the first pass that supplies prev_amax writes BF16
        w = GemmWorkload(name, 8192 // s, 4096 // s, 14336 // s, capi.E5M2, capi.E4M3, capi.BF16 if first else capi.E5M2,
                         dev, a_std=1e-3, a_scaling="outer", b_uniform=0.02, b_scaling="tensor", bias_std=0.01,
                         want_amax=True, seed=2000)
        return w
    if name in ("c3n1", "c3n8"):    # decode GEMV: W 8192^2 E5M2 row-wise, x BF16, batch 1 / 8
        nb = 1 if name == "c3n1" else 8
        w = GemmWorkload(name, 8192 // s, nb, 8192 // s, capi.E5M2, capi.BF16, capi.BF16, dev, a_std=0.02,
                         a_scaling="outer", b_std=1.0, seed=3000)
        w.units = float(w.m) * w.k + 2.0 * w.k * nb + 4.0 * w.m + 2.0 * w.m * nb
        w.unit_name = "B"
        return w
    if name == "c4":      # wgrad: E5M2 gradient (scale 1) x BF16 activations, accumulated into FP32 main_grad
        return GemmWorkload("c4", 4096 // s, 4096 // s, 65536 // s, capi.E5M2, capi.BF16, capi.FP32, dev, a_std=1e-3,
                            a_scale_inv=1.0, b_std=1.0, beta=1.0, d0_std=1e-4, seed=4000)
    if name in GEMM_ROWS:  # the rows of the reference's GEMM benchmark (bench/bench_gemm.cu:33-70): M = N = K = 4096, C1's values
        ta, tb, bt, dt, beta = GEMM_ROWS[name][1:]
        return GemmWorkload(name, 4096 // s, 4096 // s, 4096 // s, capi.E5M2, bt, dt, dev, a_std=8.0, a_scale_inv=0.125,
                            b_std=8.0 if bt in FP8_MAX else 1.0, b_scale_inv=0.125 if bt in FP8_MAX else 1.0, beta=beta,
                            d0_std=1e-2 if beta else None, seed=7000, transa=ta, transb=tb)
    if name in GEMV_ROWS:  # the rows of the reference's GEMV benchmark (bench/bench_gemv.cu:38-47): C3's weights, x in three formats
        xt, nb = GEMV_ROWS[name][1:]
        w = GemmWorkload(name, 8192 // s, nb, 8192 // s, capi.E5M2, xt, capi.BF16, dev, a_std=0.02, a_scaling="outer",
                         b_std=1.0, b_scaling="tensor", seed=3000)
        w.units = float(w.m) * w.k + float(w.B.element_size()) * w.k * nb + 4.0 * w.m + 2.0 * w.m * nb
        w.unit_name = "B"
        return w
    if name == "c5":      # AdamW over 2^30 BF16 parameters with an E4M3 copy
        return AdamWorkload("c5", (1 << 30) // s, dev, seed=5000)
    if name == "cast_f32_e5m2":
        return CastWorkload(name, (1 << 29) // s, capi.FP32, capi.E5M2, dev, seed=6000)
    if name == "cast_bf16_e4m3":
        return CastWorkload(name, (1 << 30) // s, capi.BF16, capi.E4M3, dev, seed=6100)
    if name == "cast_e4m3_bf16":
        return CastWorkload(name, (1 << 30) // s, capi.E4M3, capi.BF16, dev, seed=6200)
    raise ValueError(f"unknown workload {name}")


def finish_c2(w, prev_amax):
    """Second-pass set-up of c2: E5M2 output quantised with scale = 57344 / prev_amax."""
    w.d_scale = torch.tensor([57344.0 / max(prev_amax, 1e-30)], dtype=torch.float32, device=w.dev)
    w.amax.zero_()
    return w


# name -> (description, transa, transb, B dtype, D dtype, beta): the rows of the reference's GEMM benchmark
GEMM_ROWS = {
    "row_tn": ("e5ma_gemm TN E5M2 x E5M2 -> BF16", "T", "N", capi.E5M2, capi.BF16, 0.0),
    "row_nn": ("e5ma_gemm NN E5M2 x E5M2 -> BF16", "N", "N", capi.E5M2, capi.BF16, 0.0),
    "row_nt": ("e5ma_gemm NT E5M2 x E5M2 -> BF16", "N", "T", capi.E5M2, capi.BF16, 0.0),
    "row_tt": ("e5ma_gemm TT E5M2 x E5M2 -> BF16", "T", "T", capi.E5M2, capi.BF16, 0.0),
    "row_tn_e4m3": ("e5ma_gemm TN E5M2 x E4M3 -> BF16", "T", "N", capi.E4M3, capi.BF16, 0.0),
    "row_tn_bf16": ("e5ma_gemm TN E5M2 x BF16 -> BF16", "T", "N", capi.BF16, capi.BF16, 0.0),
    "row_tn_f32": ("e5ma_gemm TN E5M2 x FP32 -> BF16", "T", "N", capi.FP32, capi.BF16, 0.0),
    "row_tn_bf16_acc": ("e5ma_gemm TN E5M2 x BF16, FP32 D += (accumulate)", "T", "N", capi.BF16, capi.FP32, 1.0),
}

# name -> (description, x dtype, batch): the rows of the reference's GEMV benchmark
GEMV_ROWS = {f"gemv_{xn.lower()}_n{nb}": (f"e5ma gemv n={nb} x={xn} -> BF16", xt, nb)
             for xn, xt in (("E5M2", capi.E5M2), ("BF16", capi.BF16), ("FP32", capi.FP32)) for nb in (1, 2, 4, 8)}

NAMES = ["c1", "c2", "c3n1", "c3n8", "c4", "c5", "cast_f32_e5m2", "cast_bf16_e4m3", "cast_e4m3_bf16"]
