"""Host-side checks that need no GPU: the shared library loads and exports every symbol that
include/e5m2effma.h declares, structure layouts match the reference ABI, and every validation
branch returns the documented status before any device work (the order of reference
src/gemm_e5m2effma.cu:55-81, src/e5m2effma.cu:89-94, src/adamw_e5m2effma.cu:131-146)."""
import ctypes
import os
import re

import pytest

from e5m2effma_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
P = 0x1000  # a fake, 16-byte aligned, non-NULL device address; validation never dereferences it


def T(dtype, data=P, **kw):
    return capi.tensor(data, dtype, **kw)


def test_every_declared_symbol_is_exported():
    names = set()
    for fn in os.listdir(os.path.join(ROOT, "include")):
        text = open(os.path.join(ROOT, "include", fn)).read()
        names |= set(re.findall(r"\b(e5(?:ma|b)_[a-z_0-9]+)\s*\(", text))
    assert {"e5ma_gemm", "e5ma_cast", "e5ma_adam", "e5ma_status_string", "e5ma_last_error", "e5b_gemm_fault",
            "e5b_adam_multi", "e5b_set_option", "e5b_last_route"} <= names
    for n in names:
        assert hasattr(capi.lib, n), n


def test_struct_layout_matches_reference_abi():
    assert ctypes.sizeof(capi.Tensor) == 48
    assert [getattr(capi.Tensor, f).offset for f in ("data", "dtype", "scale_inv", "scale", "amax", "scaling")] == \
        [0, 8, 16, 24, 32, 40]
    assert ctypes.sizeof(capi.AdamConfig) == 36
    assert capi.AdamConfig.step.offset == 20 and capi.AdamConfig.grad_scale.offset == 32


def test_status_strings():
    assert [capi.status_string(i) for i in range(4)] == ["E5MA_OK", "E5MA_INVALID_VALUE", "E5MA_NOT_SUPPORTED", "E5MA_CUDA_ERROR"]
    assert capi.status_string(77) == "unknown e5ma_status"


def gemm(ta=1, tb=0, m=32, n=32, k=32, A=None, lda=32, B=None, ldb=32, beta=0.0, C=None, ldc=32, D=None, ldd=32,
         bias=None, alpha=1.0):
    A = T(capi.E5M2) if A is None else A
    B = T(capi.E5M2) if B is None else B
    D = T(capi.BF16) if D is None else D
    return capi.gemm(ta, tb, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc, D, ldd, bias)


GEMM_REJECTS = [
    (dict(A=T(capi.E5M2, data=None)), capi.INVALID_VALUE, "NULL"),
    (dict(ta=2), capi.INVALID_VALUE, "transa / transb"),
    (dict(m=-1), capi.INVALID_VALUE, "negative size"),
    (dict(D=T(7)), capi.INVALID_VALUE, "invalid D dtype 7"),
    (dict(A=T(capi.FP16)), capi.NOT_SUPPORTED, "E5M2, E4M3, BF16 or FP32"),
    (dict(k=24, lda=32), capi.INVALID_VALUE, "k = 24 is not a multiple of 16"),
    (dict(lda=40), capi.INVALID_VALUE, "must be multiples of 16"),
    (dict(A=T(capi.E5M2, data=P + 8)), capi.INVALID_VALUE, "16-byte aligned"),
    (dict(k=64, lda=32, ldb=64), capi.INVALID_VALUE, "lda = 32 < 64"),
    (dict(ta=0, m=48, lda=32, ldd=48), capi.INVALID_VALUE, "lda = 32 < 48"),
    (dict(tb=1, n=48, ldb=32), capi.INVALID_VALUE, "ldb = 32 < 48"),
    (dict(ldd=31), capi.INVALID_VALUE, "ldd = 31 < m = 32"),
    (dict(bias=T(9)), capi.INVALID_VALUE, "invalid bias dtype 9"),
    (dict(beta=1.0, C=T(-1)), capi.INVALID_VALUE, "invalid C dtype"),
    (dict(beta=1.0, C=T(capi.FP32), ldc=8), capi.INVALID_VALUE, "ldc = 8 < m = 32"),
    (dict(A=T(capi.E5M2, scaling=5)), capi.INVALID_VALUE, "invalid scaling of A or B"),
    (dict(A=T(capi.E5M2, scaling=1)), capi.INVALID_VALUE, "E5MA_SCALING_OUTER needs"),
    (dict(B=T(capi.BF16, scale_inv=P, scaling=1)), capi.INVALID_VALUE, "E5MA_SCALING_OUTER needs"),
    (dict(D=T(capi.BF16, scaling=1)), capi.INVALID_VALUE, "per-tensor scaling only"),
]


@pytest.mark.parametrize("kw,status,msg", GEMM_REJECTS)
def test_gemm_rejects_before_touching_the_device(kw, status, msg):
    assert gemm(**kw) == status
    assert msg in capi.last_error(), capi.last_error()
    assert capi.last_error().startswith("e5ma_gemm: ")


def test_gemm_empty_problem_succeeds_and_clears_the_error():
    assert gemm(m=-1) == capi.INVALID_VALUE and capi.last_error()
    assert gemm(m=0) == capi.OK and capi.last_error() == ""
    assert gemm(n=0, k=17) == capi.OK   # size checks come after the empty-problem exit
    assert capi.gemm(1, 0, 1, 1, 16, 1.0, None, 16, None, 16, 0.0, None, 0, None, 1, None) == capi.INVALID_VALUE


def test_cast_rejects():
    assert capi.cast(None, T(capi.BF16), 4) == capi.INVALID_VALUE and "NULL" in capi.last_error()
    assert capi.cast(T(capi.FP32), T(capi.BF16, data=None), 4) == capi.INVALID_VALUE
    assert capi.cast(T(5), T(capi.BF16), 4) == capi.INVALID_VALUE and "invalid dtype (src 5, dst 1)" in capi.last_error()
    assert capi.cast(T(capi.FP32), T(capi.E5M2, scaling=1), 4) == capi.INVALID_VALUE and "per-tensor" in capi.last_error()
    assert capi.cast(T(capi.FP32), T(capi.E5M2), 0) == capi.OK and capi.last_error() == ""


def adam_cfg(**kw):
    d = dict(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, step=1, adamw=1, bias_correction=1, grad_scale=1.0)
    d.update(kw)
    return capi.AdamConfig(*[d[f[0]] for f in capi.AdamConfig._fields_])


def test_adam_rejects():
    f32, bf = T(capi.FP32), T(capi.BF16)
    assert capi.adam(None, 8, f32, f32, f32, f32) == capi.INVALID_VALUE and "NULL" in capi.last_error()
    assert capi.adam(adam_cfg(step=0), 8, f32, f32, f32, f32) == capi.INVALID_VALUE and "step = 0" in capi.last_error()
    assert capi.adam(adam_cfg(), 8, T(capi.FP16), f32, f32, f32) == capi.NOT_SUPPORTED
    assert capi.adam(adam_cfg(), 8, f32, f32, f32, bf) == capi.NOT_SUPPORTED and "both" in capi.last_error()
    assert capi.adam(adam_cfg(), 8, f32, T(capi.E5M2), f32, f32) == capi.NOT_SUPPORTED and "grad" in capi.last_error()
    assert capi.adam(adam_cfg(), 8, f32, f32, f32, f32, T(capi.BF16)) == capi.INVALID_VALUE and "param_fp8" in capi.last_error()
    assert capi.adam(adam_cfg(), 8, f32, f32, f32, f32, T(capi.E4M3, scaling=1)) == capi.INVALID_VALUE
    assert capi.adam(adam_cfg(), 0, f32, f32, f32, f32) == capi.OK and capi.last_error() == ""


def test_no_device_gives_an_error_not_a_fallback():
    """Without a usable sm_100 device a valid call fails with a status; nothing is computed on the CPU."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    st = gemm()
    assert st in (capi.CUDA_ERROR, capi.NOT_SUPPORTED) and capi.last_error()


def test_adam_multi_rejects():
    f32, bf = T(capi.FP32), T(capi.BF16)
    cfg = adam_cfg()
    assert capi.adam_multi(None, [8], [f32], [f32], [f32], [f32]) == capi.INVALID_VALUE
    assert capi.adam_multi(adam_cfg(step=0), [8], [f32], [f32], [f32], [f32]) == capi.INVALID_VALUE
    assert capi.adam_multi(cfg, [8], [T(capi.FP16)], [f32], [f32], [f32]) == capi.NOT_SUPPORTED
    assert capi.adam_multi(cfg, [8, 8], [f32, bf], [f32, f32], [f32, f32], [f32, f32]) == capi.INVALID_VALUE
    assert "differs in dtype" in capi.last_error()
    assert capi.adam_multi(cfg, [8], [T(capi.FP32, data=None)], [f32], [f32], [f32]) == capi.INVALID_VALUE
    assert capi.adam_multi(cfg, [], [], [], [], []) == capi.OK and capi.last_error() == ""


def test_options_and_route_record():
    """e5b_set_option knows every documented switch (with or without the E5MA_ prefix), rejects others, and the
    route record starts at 'none' and stays there for calls that launch nothing."""
    for name in ["FORCE_SIMT", "TC_PAIR", "TC_SPLIT", "TC_GRID", "TC_WIDE", "GEMV_KERNEL", "GEMV_STAGES", "GEMV_U",
                 "GEMV_MT", "MIXED_PAIR", "E5MA_TC_PAIR"]:
        capi.set_option(name, 1)
        capi.set_option(name, None)
    with pytest.raises(KeyError):
        capi.set_option("NO_SUCH_SWITCH", 1)
    t = capi.tensor(16, capi.E5M2)
    assert capi.gemm(capi.OP_T, capi.OP_N, 0, 4, 16, 1.0, t, 16, t, 16, 0.0, None, 0, capi.tensor(16, capi.BF16), 1, None) == capi.OK
    assert capi.last_route() == capi.ROUTE_NONE


def test_peer_barrier_rejects_bad_arguments():
    flags = (ctypes.c_void_p * 8)(*([0x1000] * 8))
    assert capi.lib.e5b_peer_barrier(0, 0, flags, None) == capi.INVALID_VALUE
    assert capi.lib.e5b_peer_barrier(0, 9, flags, None) == capi.INVALID_VALUE
    assert capi.lib.e5b_peer_barrier(2, 2, flags, None) == capi.INVALID_VALUE and "rank 2 of 2" in capi.last_error()
    assert capi.lib.e5b_peer_barrier(0, 2, None, None) == capi.INVALID_VALUE
    flags[1] = 0
    assert capi.lib.e5b_peer_barrier(0, 2, flags, None) == capi.INVALID_VALUE and "flags[1]" in capi.last_error()
    flags[1] = 0x1002
    assert capi.lib.e5b_peer_barrier(0, 2, flags, None) == capi.INVALID_VALUE
