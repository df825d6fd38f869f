"""ctypes face of the CPU oracle (oracle/oracle.cpp) -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Only tests/, the smoke check and the cpu_baseline / reference legs of bench.py import this
module.  Arrays are numpy; storage dtypes are uint8 for the two FP8 formats, uint16 for BF16
and FP16 bit patterns and float32 for FP32.  dtype codes are those of include/e5m2effma.h.
"""
import ctypes
import os
import subprocess

import numpy as np

E4M3, BF16, FP16, FP32, E5M2 = 0, 1, 2, 3, 4
NP_STORAGE = {E4M3: np.uint8, E5M2: np.uint8, BF16: np.uint16, FP16: np.uint16, FP32: np.float32}
_HERE = os.path.dirname(os.path.abspath(__file__))


def build():
    """Compile liboracle.so (and oracle/_ref when the reference sources are present)."""
    subprocess.run(["make", "-s", "-C", _HERE], check=True)


def usable_cpus():
    """CPUs this process may really use: the affinity mask, cut down to the cgroup CPU quota.
    OpenMP defaults to every CPU of the host, which stalls badly inside a CPU-limited container."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    try:
        quota, period = open("/sys/fs/cgroup/cpu.max").read().split()
        if quota != "max":
            n = min(n, max(1, int(float(quota) / float(period))))
    except (OSError, ValueError):
        try:
            q = int(open("/sys/fs/cgroup/cpu/cpu.cfs_quota_us").read())
            per = int(open("/sys/fs/cgroup/cpu/cpu.cfs_period_us").read())
            if q > 0 and per > 0:
                n = min(n, max(1, q // per))
        except (OSError, ValueError):
            pass
    return max(1, n)


def _load():
    path = os.path.join(_HERE, "liboracle.so")
    if not os.path.exists(path):
        build()
    os.environ.setdefault("OMP_WAIT_POLICY", "passive")   # idle workers sleep instead of spinning
    return ctypes.CDLL(path)


_lib = _load()
_f = ctypes.c_float
_p = ctypes.c_void_p
_fp = ctypes.POINTER(ctypes.c_float)


class GemmArgs(ctypes.Structure):
    _fields_ = [
        ("transa", ctypes.c_int), ("transb", ctypes.c_int), ("m", ctypes.c_int), ("n", ctypes.c_int),
        ("k", ctypes.c_int), ("alpha", _f), ("beta", _f),
        ("a", _p), ("a_dtype", ctypes.c_int), ("a_sinv", _p), ("a_outer", ctypes.c_int), ("lda", ctypes.c_int),
        ("b", _p), ("b_dtype", ctypes.c_int), ("b_sinv", _p), ("b_outer", ctypes.c_int), ("ldb", ctypes.c_int),
        ("c", _p), ("c_dtype", ctypes.c_int), ("c_sinv", _p), ("ldc", ctypes.c_int),
        ("d", _p), ("d_dtype", ctypes.c_int), ("d_scale", _p), ("ldd", ctypes.c_int),
        ("bias", _p), ("bias_dtype", ctypes.c_int),
        ("amax", _p),
    ]


class AdamCfg(ctypes.Structure):
    _fields_ = [("lr", _f), ("beta1", _f), ("beta2", _f), ("eps", _f), ("weight_decay", _f),
                ("step", ctypes.c_int), ("adamw", ctypes.c_int), ("bias_correction", ctypes.c_int),
                ("grad_scale", _f)]


_lib.orc_threads.restype = ctypes.c_int
_lib.orc_set_threads.argtypes = [ctypes.c_int]
_lib.orc_set_threads.restype = None
_lib.orc_decode_n.argtypes = [ctypes.c_int, _p, ctypes.c_size_t, _f, _p]
_lib.orc_encode_n.argtypes = [ctypes.c_int, _p, ctypes.c_size_t, _p, _f]
_lib.orc_lane.argtypes = [ctypes.c_uint32] * 3 + [ctypes.c_int] * 2
_lib.orc_lane.restype = ctypes.c_uint32
_lib.orc_lane_n.argtypes = [ctypes.c_size_t, _p, _p, _p, ctypes.c_int, ctypes.c_int, _p]
_lib.orc_cast.argtypes = [ctypes.c_int, _p, ctypes.c_int, _p, ctypes.c_size_t, _p, _p, _p]
_lib.orc_gemm_cols.argtypes = [ctypes.POINTER(GemmArgs), ctypes.c_int, ctypes.c_int, ctypes.c_int]
_lib.orc_gemm_wide.argtypes = [ctypes.POINTER(GemmArgs), ctypes.c_int, ctypes.c_int, _p, _p, _p]
_lib.orc_adam.argtypes = [ctypes.POINTER(AdamCfg), ctypes.c_size_t, _p, ctypes.c_int, _p, ctypes.c_int, _p, _p,
                          ctypes.c_int, _p, ctypes.c_int, _p, _p]


def threads():
    return _lib.orc_threads()


_lib.orc_set_threads(min(usable_cpus(), 64))


def set_threads(n):
    _lib.orc_set_threads(int(n))


def _ptr(a):
    return None if a is None else a.ctypes.data_as(_p)


def _f32(x):
    """A python float or numpy array as a C-contiguous float32 array (or None)."""
    if x is None:
        return None
    return np.ascontiguousarray(np.asarray(x, dtype=np.float32).reshape(-1))


def esize(dtype):
    return np.dtype(NP_STORAGE[dtype]).itemsize


def decode(dtype, raw, scale_inv=1.0):
    """Typed storage -> float32 values (FP8 values times scale_inv, one FP32 multiply)."""
    raw = np.ascontiguousarray(raw)
    assert raw.dtype == NP_STORAGE[dtype], (raw.dtype, dtype)
    out = np.empty(raw.size, np.float32)
    _lib.orc_decode_n(dtype, _ptr(raw), raw.size, float(scale_inv), _ptr(out))
    return out.reshape(raw.shape)


def encode(dtype, values, scale=1.0):
    """float32 values -> typed storage (FP8: saturating RNE of value * scale)."""
    v = np.ascontiguousarray(values, dtype=np.float32)
    out = np.empty(v.shape, NP_STORAGE[dtype])
    _lib.orc_encode_n(dtype, _ptr(out), v.size, _ptr(v), float(scale))
    return out


def lane(a, b, acc, fa, fb):
    """RN_BF16(acc + a*b); fa/fb: 0 = E4M3, 1 = E5M2; acc and result are BF16 bit patterns."""
    return _lib.orc_lane(int(a), int(b), int(acc), int(fa), int(fb))


def lane_n(a, b, acc, fa, fb):
    a, b, acc = (np.ascontiguousarray(x, dtype=np.uint32) for x in (a, b, acc))
    out = np.empty(a.size, np.uint32)
    _lib.orc_lane_n(a.size, _ptr(a), _ptr(b), _ptr(acc), int(fa), int(fb), _ptr(out))
    return out


def cast(src, sdt, ddt, scale_inv=None, scale=None, amax=None):
    """Returns (dst storage array, amax after the max-reduction into `amax`, or None)."""
    src = np.ascontiguousarray(src)
    assert src.dtype == NP_STORAGE[sdt]
    dst = np.empty(src.shape, NP_STORAGE[ddt])
    si, sc = _f32(scale_inv), _f32(scale)
    am = None if amax is None else np.array([amax], np.float32)
    _lib.orc_cast(sdt, _ptr(src), ddt, _ptr(dst), src.size, _ptr(si), _ptr(sc), _ptr(am))
    return dst, (None if am is None else am[0])


def _gemm_args(transa, transb, m, n, k, alpha, A, a_dtype, lda, B, b_dtype, ldb, beta, C, c_dtype, ldc,
               D, d_dtype, ldd, bias, bias_dtype, a_sinv, a_outer, b_sinv, b_outer, c_sinv, d_scale, amax_arr):
    keep = [A, B, C, D, bias, _f32(a_sinv), _f32(b_sinv), _f32(c_sinv), _f32(d_scale), amax_arr]
    g = GemmArgs(int(transa), int(transb), m, n, k, float(alpha), float(beta),
                 _ptr(A), a_dtype, _ptr(keep[5]), int(bool(a_outer)), lda,
                 _ptr(B), b_dtype, _ptr(keep[6]), int(bool(b_outer)), ldb,
                 _ptr(C), c_dtype if C is not None else FP32, _ptr(keep[7]), ldc,
                 _ptr(D), d_dtype, _ptr(keep[8]), ldd,
                 _ptr(bias), bias_dtype if bias is not None else FP32,
                 _ptr(amax_arr))
    return g, keep


def gemm(transa, transb, m, n, k, alpha, A, a_dtype, lda, B, b_dtype, ldb, beta, C, c_dtype, ldc,
         D, d_dtype, ldd, bias=None, bias_dtype=FP32, a_sinv=None, a_outer=False, b_sinv=None,
         b_outer=False, c_sinv=None, d_scale=None, amax=None, order=0, cols=None):
    """Host emulation of e5ma_gemm in the reference's operation order.

    A, B, C, D, bias are flat numpy storage arrays laid out exactly as the device buffers
    (column-major with the given leading dimensions).  D is updated in place (pass a copy);
    for accumulate mode pass C = a copy of D's initial content, c_dtype = d_dtype, ldc = ldd.
    order 0: ascending-k FMA chain; order 1: the reference GEMV kernel's lane order.
    Returns the amax value after max-reduction into `amax` (None when amax is None).
    """
    am = None if amax is None else np.array([amax], np.float32)
    g, keep = _gemm_args(transa, transb, m, n, k, alpha, A, a_dtype, lda, B, b_dtype, ldb, beta, C, c_dtype, ldc,
                         D, d_dtype, ldd, bias, bias_dtype, a_sinv, a_outer, b_sinv, b_outer, c_sinv, d_scale, am)
    j0, j1 = (0, n) if cols is None else cols
    _lib.orc_gemm_cols(ctypes.byref(g), int(order), j0, j1)
    del keep
    return None if am is None else am[0]


def gemm_wide(transa, transb, m, n, k, alpha, A, a_dtype, lda, B, b_dtype, ldb, beta, C, c_dtype, ldc,
              bias=None, bias_dtype=FP32, a_sinv=None, a_outer=False, b_sinv=None, b_outer=False,
              c_sinv=None, cols=None):
    """Double-precision epilogue value, sum |a*b|*|s| and |bias|+|beta*C| per output of the
    columns [j0, j1): three float64 arrays of shape (j1-j0, m)."""
    j0, j1 = (0, n) if cols is None else cols
    g, keep = _gemm_args(transa, transb, m, n, k, alpha, A, a_dtype, lda, B, b_dtype, ldb, beta, C, c_dtype, ldc,
                         None, FP32, m, bias, bias_dtype, a_sinv, a_outer, b_sinv, b_outer, c_sinv, None, None)
    ref = np.empty((j1 - j0, m), np.float64)
    mag = np.empty_like(ref)
    fix = np.empty_like(ref)
    _lib.orc_gemm_wide(ctypes.byref(g), j0, j1, _ptr(ref), _ptr(mag), _ptr(fix))
    del keep
    return ref, mag, fix


def adam(cfg, p, pt, g, gt, m, v, mt, q=None, qt=E4M3, qscale=None, amax=None):
    """In-place Adam / AdamW step on numpy storage arrays; cfg is a dict with the fields of
    e5ma_adam_config.  Returns amax after the max-reduction (None when not requested)."""
    c = AdamCfg(cfg["lr"], cfg["beta1"], cfg["beta2"], cfg["eps"], cfg["weight_decay"], cfg["step"],
                cfg["adamw"], cfg["bias_correction"], cfg["grad_scale"])
    qs = _f32(qscale)
    am = None if amax is None else np.array([amax], np.float32)
    _lib.orc_adam(ctypes.byref(c), p.size, _ptr(p), pt, _ptr(g), gt, _ptr(m), _ptr(v), mt, _ptr(q), qt, _ptr(qs),
                  _ptr(am))
    return None if am is None else am[0]
