"""e5ma_adam on the GPU against the oracle, bit for bit (stricter than the 1-ulp bound asked for):
the 12 dtype combinations, Adam and AdamW, steps 1..9, FP8 copy + amax, a tail after the 8-element
groups and unaligned gradients -- the matrix of reference tests/test_adamw.cu:9-61."""
import numpy as np
import pytest

import oracle as orc
from harness import BF16, E4M3, E5M2, FP16, FP32, fill, from_dev, to_dev

pytestmark = pytest.mark.gpu


def run(pt, gt, mt, qt, adamw, step, unaligned=False, n=100003, with_copy=True):
    import torch
    from e5m2effma_b200 import capi
    rng = np.random.default_rng(pt * 100 + gt * 10 + mt + step)
    cfg = dict(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, step=step, adamw=adamw,
               bias_correction=1, grad_scale=0.5)
    p = fill(pt, n, 1.0, rng); g = fill(gt, n, 0.1, rng); m = fill(mt, n, 0.01, rng)
    v = orc.encode(mt, np.abs(orc.decode(mt, m)) * np.float32(0.01))
    off = orc.esize(gt) if unaligned else 0
    bp, pp = to_dev(p); bg, pg = to_dev(g, off); bm, pm = to_dev(m); bv, pv = to_dev(v)
    bq, pq = to_dev(np.full(n + 16, 0xA5, np.uint8)); bs, ps = to_dev(np.array([64.0], np.float32))
    ba, pa = to_dev(np.zeros(1, np.float32))
    c = capi.AdamConfig(*[cfg[f[0]] for f in capi.AdamConfig._fields_])
    Q = capi.tensor(pq, qt, None, ps, pa) if with_copy else None
    st = capi.adam(c, n, capi.tensor(pp, pt), capi.tensor(pg, gt), capi.tensor(pm, mt), capi.tensor(pv, mt), Q,
                   torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert st == capi.OK, capi.last_error()
    ep, em, ev = p.copy(), m.copy(), v.copy()
    eq = np.zeros(n, np.uint8)
    eam = orc.adam(cfg, ep, pt, g, gt, em, ev, mt, eq if with_copy else None, qt, 64.0, 0.0 if with_copy else None)
    S = orc.NP_STORAGE
    def eq_bits(a, b):
        return np.array_equal(a.view(np.uint8), b.view(np.uint8))
    assert eq_bits(from_dev(bp, S[pt], n), ep), "param"
    assert eq_bits(from_dev(bm, S[mt], n), em), "exp_avg"
    assert eq_bits(from_dev(bv, S[mt], n), ev), "exp_avg_sq"
    q = from_dev(bq, np.uint8, n + 16)
    assert (q[n:] == 0xA5).all()
    if with_copy:
        assert np.array_equal(q[:n], eq), "fp8 copy"
        assert from_dev(ba, np.float32, 1)[0] == eam
    else:
        assert (q == 0xA5).all() and from_dev(ba, np.float32, 1)[0] == 0.0


@pytest.mark.parametrize("pt", [FP32, BF16])
@pytest.mark.parametrize("gt", [FP32, BF16, FP16])
@pytest.mark.parametrize("mt", [FP32, BF16])
def test_adam_combination(pt, gt, mt):
    run(pt, gt, mt, E4M3 if (pt + mt) & 1 else E5M2, (pt + gt + mt) & 1, 1 + (gt * 3 + mt))


def test_adam_unaligned_gradient():
    run(FP32, BF16, FP32, E5M2, 1, 3, unaligned=True)
    run(BF16, FP16, BF16, E4M3, 0, 4, unaligned=True)


def test_adam_without_copy_leaves_amax_alone():
    run(BF16, BF16, BF16, E4M3, 1, 2, with_copy=False)


@pytest.mark.parametrize("n", [1, 7, 8, 9, 2048 * 8 + 5])
def test_adam_small_counts(n):
    run(BF16, BF16, BF16, E4M3, 1, 1, n=n)


def test_adamw_multi_step_matches_torch_closely():
    """Five steps against torch.optim.AdamW in FP32 (the reference's binding test, lines 128-142)."""
    import torch
    import e5m2effma_b200 as fx
    torch.manual_seed(0)
    p0 = torch.randn(10007, device="cuda")
    p1 = p0.clone().requires_grad_(True)
    opt = torch.optim.AdamW([p1], lr=1e-2, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.1)
    p, m, v = p0.clone(), torch.zeros_like(p0), torch.zeros_like(p0)
    for step in range(1, 6):
        g = torch.randn_like(p0)
        p1.grad = g.clone()
        opt.step()
        fx.adam_step(p, g, m, v, lr=1e-2, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.1, step=step)
    assert torch.allclose(p, p1.detach(), rtol=2e-5, atol=2e-6)
