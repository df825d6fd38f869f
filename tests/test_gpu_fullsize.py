"""Parity at the full benchmark sizes (BASELINE.json configs), on seeded synthetic inputs generated
on the GPU: the GEMM configurations are checked on sampled output columns at full K (every row of
those columns) against the oracle with the stated tolerance; the GEMV and the 4096^3 GEMM on the
whole output; AdamW and a cast on sampled chunks, bit for bit (element-wise operations: a chunk is
as good as the whole)."""
import numpy as np
import pytest

import oracle as orc
from harness import ordered

pytestmark = pytest.mark.gpu


def _host(t):
    import torch
    return t.detach().cpu().contiguous().view(torch.uint8).numpy()


def _check_columns(w, cols, k_eps=1.0):
    """Compares columns `cols` (list of (j0, j1)) of the device result w.D with the oracle."""
    import torch
    from e5m2effma_b200 import capi
    es = {capi.BF16: np.uint16, capi.FP32: np.float32, capi.E5M2: np.uint8, capi.E4M3: np.uint8}
    A = _host(w.A).view(es[w.a_dtype]).reshape(-1)
    B = _host(w.B).view(es[w.b_dtype]).reshape(-1)
    sa = None if w.sa is None else w.sa.cpu().numpy()
    sb = None if w.sb is None else w.sb.cpu().numpy()
    bias = None if w.bias is None else _host(w.bias).view(np.uint16)
    D = _host(w.D).view(es[w.d_dtype]).reshape(w.n, w.m)
    C0 = None if w.D0 is None else _host(w.D0).view(es[w.d_dtype]).reshape(-1)
    qs = float(w.d_scale.item()) if w.d_scale is not None else 1.0
    amax_seen = 0.0
    for j0, j1 in cols:
        ref, mag, fix = orc.gemm_wide(int(w.transa == "T"), int(w.transb == "T"), w.m, w.n, w.k, 1.0, A, w.a_dtype, w.lda, B, w.b_dtype, w.ldb, w.beta, C0, w.d_dtype,
                                      w.m, bias=bias, bias_dtype=orc.BF16, a_sinv=sa, a_outer=w.a_outer, b_sinv=sb,
                                      b_outer=w.b_outer, cols=(j0, j1))
        bound = w.k * 2.0 ** -23 * mag * k_eps + 2.0 ** -21 * (np.abs(ref) + fix + mag)
        f32max = float(np.finfo(np.float32).max)
        enc = lambda v: orc.encode(w.d_dtype, np.clip(v, -f32max, f32max).astype(np.float32), qs)
        lo, hi = ordered(w.d_dtype, enc(ref - bound)), ordered(w.d_dtype, enc(ref + bound))
        got = ordered(w.d_dtype, D[j0:j1].copy())
        ok = (got >= np.minimum(lo, hi) - 1) & (got <= np.maximum(lo, hi) + 1)
        assert ok.all(), f"{w.name}: {int((~ok).sum())} outputs of columns [{j0},{j1}) outside tolerance"
        amax_seen = max(amax_seen, float(np.abs(ref).max()))
    return amax_seen


def _run(w):
    import torch
    from e5m2effma_b200 import capi
    w.launch(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert capi.gemm_fault() == 0


def test_c1_gemm_4096_cube_whole_output():
    import torch
    from e5m2effma_b200 import workloads
    w = workloads.make("c1", torch.device("cuda", 0))
    _run(w)
    _check_columns(w, [(0, 4096)])


def test_c2_hybrid_dgrad_sampled_columns():
    import torch
    from e5m2effma_b200 import capi, workloads
    dev = torch.device("cuda", 0)
    w = workloads.make("c2_bf16", dev)
    _run(w)
    prev_amax = float(w.amax.item())
    _check_columns(w, [(0, 8), (2040, 2056), (4088, 4096)])
    w.d_dtype = capi.E5M2
    w.D = torch.zeros((w.n, w.m), dtype=torch.uint8, device=dev)
    workloads.finish_c2(w, prev_amax)
    _run(w)
    seen = _check_columns(w, [(0, 8), (1000, 1016), (4088, 4096)])
    assert float(w.amax.item()) >= seen * (1 - 2.0 ** -7) and abs(float(w.amax.item()) - prev_amax) <= prev_amax * 2.0 ** -6


@pytest.mark.parametrize("name", ["c3n1", "c3n8", "gemv_e5m2_n4", "gemv_fp32_n1", "gemv_fp32_n2", "gemv_fp32_n4", "gemv_fp32_n8"])
def test_c3_decode_gemv_whole_output(name):
    import torch
    from e5m2effma_b200 import capi, workloads
    w = workloads.make(name, torch.device("cuda", 0))
    _run(w)
    assert capi.last_route() in ((capi.ROUTE_GEMV_FMA,) if w.b_dtype == capi.FP32 else (capi.ROUTE_GEMV, capi.ROUTE_GEMV_FMA, capi.ROUTE_GEMV_ROWS))
    _check_columns(w, [(0, w.n)])


def test_c4_wgrad_accumulate_sampled_columns():
    import torch
    from e5m2effma_b200 import workloads
    w = workloads.make("c4", torch.device("cuda", 0))
    _run(w)
    _check_columns(w, [(0, 4), (2046, 2050), (4092, 4096)])


@pytest.mark.parametrize("name", ["row_tn", "row_nn", "row_nt", "row_tt", "row_tn_e4m3", "row_tn_bf16", "row_tn_f32", "row_tn_bf16_acc"])
def test_reference_benchmark_rows_sampled_columns(name):
    """The 4096^3 rows of the reference's GEMM benchmark (four layouts, the pairings, accumulate mode): sampled columns
    against the oracle, and the kernel each row is expected to take."""
    import torch
    from e5m2effma_b200 import capi, workloads
    w = workloads.make(name, torch.device("cuda", 0))
    _run(w)
    expected = {"row_tn": (capi.ROUTE_TC_PAIR, capi.ROUTE_TC_PAIR_WIDE), "row_tn_e4m3": (capi.ROUTE_TC_PAIR, capi.ROUTE_TC_PAIR_WIDE),
                "row_tn_f32": (capi.ROUTE_SIMT,)}.get(name, (capi.ROUTE_TC_256, capi.ROUTE_TC_128, capi.ROUTE_TC_256_KTAIL, capi.ROUTE_TC_128_KTAIL))
    assert capi.last_route() in expected
    _check_columns(w, [(0, 4), (2047, 2051), (4092, 4096)])


def test_the_four_layouts_of_one_problem_agree():
    """Same values stored in the four operand layouts: the outputs may differ by the order in which a tile's k-blocks
    are added (one BF16 code, rarely), nothing more."""
    import torch
    from e5m2effma_b200 import workloads
    dev = torch.device("cuda", 0)
    outs = []
    for name in ("row_tn", "row_nn", "row_nt", "row_tt"):
        w = workloads.make(name, dev, 4)
        _run(w)
        outs.append(w.D.view(torch.int16).int())
    for o in outs[1:]:
        diff = (o - outs[0]).abs()
        assert int(diff.max()) <= 1 and float((diff != 0).float().mean()) < 0.02


def test_c5_adamw_sampled_chunks_bit_exact():
    import torch
    from e5m2effma_b200 import workloads
    dev = torch.device("cuda", 0)
    w = workloads.make("c5", dev)
    n = 1 << 22
    spots = [0, (1 << 29) + 8, (1 << 30) - n]
    before = [(_host(w.p[s:s + n]).view(np.uint16).copy(), _host(w.g[s:s + n]).view(np.uint16).copy()) for s in spots]
    w.launch(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    cfg = dict(lr=3e-4, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.1, step=1, adamw=1, bias_correction=1, grad_scale=1.0)
    top = 0.0
    for s, (p, g) in zip(spots, before):
        m, v, q = np.zeros(n, np.uint16), np.zeros(n, np.uint16), np.zeros(n, np.uint8)
        top = max(top, orc.adam(cfg, p, orc.BF16, g, orc.BF16, m, v, orc.BF16, q, orc.E4M3, 2048.0, 0.0))
        assert np.array_equal(_host(w.p[s:s + n]).view(np.uint16), p)
        assert np.array_equal(_host(w.m[s:s + n]).view(np.uint16), m)
        assert np.array_equal(_host(w.v[s:s + n]).view(np.uint16), v)
        assert np.array_equal(_host(w.q[s:s + n]), q)
    assert float(w.amax.item()) >= top


def test_cast_sampled_chunks_bit_exact():
    import torch
    from e5m2effma_b200 import workloads
    w = workloads.make("cast_f32_e5m2", torch.device("cuda", 0))
    w.launch(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    n = 1 << 22
    for s in (0, (1 << 28) + 16, (1 << 29) - n):
        src = w.src[s:s + n].cpu().numpy()
        exp, _ = orc.cast(src, orc.FP32, orc.E5M2, None, 16.0)
        assert np.array_equal(_host(w.dst[s:s + n]), exp)
