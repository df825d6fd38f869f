"""ctypes declarations of the C interface in include/e5m2effma.h, bound to libe5m2effma.so.

This is the whole boundary: five entry points, plain pointers and sizes.  The library is the
sm_100a build in this directory; it is never substituted -- if it is missing the import fails.
"""
import ctypes
import os

E4M3, BF16, FP16, FP32, E5M2 = 0, 1, 2, 3, 4
OP_N, OP_T = 0, 1
OK, INVALID_VALUE, NOT_SUPPORTED, CUDA_ERROR = 0, 1, 2, 3
SCALING_TENSOR, SCALING_OUTER = 0, 1

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libe5m2effma.so")


class Tensor(ctypes.Structure):
    """e5ma_tensor: 48 bytes, fields at 0 / 8 / 16 / 24 / 32 / 40."""
    _fields_ = [("data", ctypes.c_void_p), ("dtype", ctypes.c_int), ("scale_inv", ctypes.c_void_p),
                ("scale", ctypes.c_void_p), ("amax", ctypes.c_void_p), ("scaling", ctypes.c_int)]


class AdamConfig(ctypes.Structure):
    """e5ma_adam_config: 36 bytes."""
    _fields_ = [("lr", ctypes.c_float), ("beta1", ctypes.c_float), ("beta2", ctypes.c_float),
                ("eps", ctypes.c_float), ("weight_decay", ctypes.c_float), ("step", ctypes.c_int),
                ("adamw", ctypes.c_int), ("bias_correction", ctypes.c_int), ("grad_scale", ctypes.c_float)]


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
            "or `make -C e5m2effma_b200/csrc` (needs nvcc with sm_100a support); there is no fallback path")
    lib = ctypes.CDLL(LIB_PATH)
    tp = ctypes.POINTER(Tensor)
    lib.e5ma_gemm.restype = ctypes.c_int
    lib.e5ma_gemm.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_float,
                              tp, ctypes.c_int, tp, ctypes.c_int, ctypes.c_float, tp, ctypes.c_int, tp, ctypes.c_int,
                              tp, ctypes.c_void_p]
    lib.e5ma_cast.restype = ctypes.c_int
    lib.e5ma_cast.argtypes = [tp, tp, ctypes.c_size_t, ctypes.c_void_p]
    lib.e5ma_adam.restype = ctypes.c_int
    lib.e5ma_adam.argtypes = [ctypes.POINTER(AdamConfig), ctypes.c_size_t, tp, tp, tp, tp, tp, ctypes.c_void_p]
    lib.e5ma_status_string.restype = ctypes.c_char_p
    lib.e5ma_status_string.argtypes = [ctypes.c_int]
    lib.e5ma_last_error.restype = ctypes.c_char_p
    lib.e5ma_last_error.argtypes = []
    lib.e5b_gemm_fault.restype = ctypes.c_uint
    lib.e5b_gemm_fault.argtypes = []
    lib.e5b_peer_barrier.restype = ctypes.c_int
    lib.e5b_peer_barrier.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p]
    lib.e5b_gemm_bcast.restype = ctypes.c_int
    lib.e5b_gemm_bcast.argtypes = lib.e5ma_gemm.argtypes[:-1] + [ctypes.c_int, ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p]
    lib.e5b_set_option.restype = ctypes.c_int
    lib.e5b_set_option.argtypes = [ctypes.c_char_p, ctypes.c_int]
    lib.e5b_tuned_plan.restype = ctypes.c_int
    lib.e5b_tuned_plan.argtypes = [ctypes.c_int] * 4
    lib.e5b_last_route.restype = ctypes.c_int
    lib.e5b_last_route.argtypes = []
    lib.e5b_adam_multi.restype = ctypes.c_int
    lib.e5b_adam_multi.argtypes = [ctypes.POINTER(AdamConfig), ctypes.c_int, ctypes.POINTER(ctypes.c_size_t), tp, tp, tp, tp, tp,
                                   ctypes.c_void_p]
    return lib


lib = _load()


def status_string(status):
    return lib.e5ma_status_string(int(status)).decode()


def last_error():
    return lib.e5ma_last_error().decode()


def gemm_fault():
    """Fault record of the tensor-core GEMM (0 = none); synchronises and clears it."""
    return int(lib.e5b_gemm_fault())


ROUTE_NONE, ROUTE_GEMV, ROUTE_GEMV_PERSISTENT, ROUTE_TC_PAIR, ROUTE_TC_PAIR_WIDE, ROUTE_TC_256, ROUTE_TC_128, ROUTE_SIMT, \
    ROUTE_TC_MIXED_PAIR, ROUTE_GEMV_FMA, ROUTE_GEMV_ROWS, ROUTE_TC_256_KSPLIT, ROUTE_TC_128_KSPLIT, \
    ROUTE_TC_256_KTAIL, ROUTE_TC_128_KTAIL = range(15)


def set_option(name, value):
    """e5b_set_option: kernel-selection switch `name` (e.g. "TC_PAIR") = value; None or a negative value restores
    the library's own choice."""
    if lib.e5b_set_option(name.encode(), -1 if value is None else int(value)) != 0:
        raise KeyError(f"unknown option {name}")


def tuned_plan(elem_bytes, m, n, k):
    """Tuned-table plan of a GEMM problem (-2: no entry); see e5b_tuned_plan."""
    return int(lib.e5b_tuned_plan(elem_bytes, m, n, k))


def last_route():
    """Which kernel the last gemm() call of this thread launched (ROUTE_*)."""
    return int(lib.e5b_last_route())


def tensor(data, dtype, scale_inv=None, scale=None, amax=None, scaling=SCALING_TENSOR):
    """Builds an e5ma_tensor from raw device addresses (ints or None)."""
    return Tensor(data, dtype, scale_inv, scale, amax, scaling)


def _ref(t):
    return None if t is None else ctypes.byref(t)


def gemm(transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, D, ldd, bias, stream=0):
    """e5ma_gemm; tensors are capi.Tensor (or None); returns the e5ma_status."""
    return lib.e5ma_gemm(transa, transb, m, n, k, alpha, _ref(A), lda, _ref(B), ldb, beta, _ref(C), ldc, _ref(D), ldd,
                         _ref(bias), stream)


def gemm_bcast(transa, transb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, D, ldd, bias, peers, stream=0):
    """e5b_gemm_bcast: e5ma_gemm that also stores D into the buffers whose device addresses are listed in `peers`."""
    arr = (ctypes.c_void_p * max(len(peers), 1))(*peers)
    return lib.e5b_gemm_bcast(transa, transb, m, n, k, alpha, _ref(A), lda, _ref(B), ldb, beta, _ref(C), ldc, _ref(D), ldd,
                              _ref(bias), len(peers), arr, stream)


def peer_barrier(rank, flag_ptrs, stream=0):
    """e5b_peer_barrier: device-side barrier between the ranks whose flag areas are at `flag_ptrs` (indexed by rank)."""
    arr = (ctypes.c_void_p * len(flag_ptrs))(*flag_ptrs)
    return lib.e5b_peer_barrier(rank, len(flag_ptrs), arr, stream)


def cast(src, dst, count, stream=0):
    return lib.e5ma_cast(_ref(src), _ref(dst), count, stream)


def adam(cfg, count, param, grad, exp_avg, exp_avg_sq, param_fp8=None, stream=0):
    return lib.e5ma_adam(None if cfg is None else ctypes.byref(cfg), count, _ref(param), _ref(grad), _ref(exp_avg),
                         _ref(exp_avg_sq), _ref(param_fp8), stream)


def adam_multi(cfg, counts, params, grads, exp_avgs, exp_avg_sqs, params_fp8=None, stream=0):
    """e5b_adam_multi: lists of capi.Tensor of equal length (params_fp8: None or a list whose entries may
    have data = None for "no copy"... all entries must then agree); returns the e5ma_status."""
    n = len(counts)
    arr = lambda ts: (Tensor * n)(*ts) if n else (Tensor * 1)()
    c = (ctypes.c_size_t * max(n, 1))(*counts)
    q = None if params_fp8 is None else arr(params_fp8)
    return lib.e5b_adam_multi(None if cfg is None else ctypes.byref(cfg), n, c, arr(params), arr(grads), arr(exp_avgs),
                              arr(exp_avg_sqs), q, stream)
