"""The torch-facing wrappers (e5m2effma_b200.functional) against a float64 reference, with the
bound and the cases of the reference's binding tests (binds/python/tests/test_e5m2effma.py:26-31,
43-125, 180-335): |y - ref| <= eps(out) * |ref| + k * 2^-23 * sum |a| |b|."""
import pytest
import torch

pytestmark = pytest.mark.gpu
F8, F4 = torch.float8_e5m2, torch.float8_e4m3fn
DEV = "cuda"


def fx():
    import e5m2effma_b200
    return e5m2effma_b200


def rand(shape, dtype, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(DEV).to(dtype)


def check_close(y, ref, mag, k, out_dtype):
    eps = {torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11, torch.float32: 2.0 ** -24, F8: 2.0 ** -3, F4: 2.0 ** -4}[out_dtype]
    err = (y.double() - ref).abs()
    bound = eps * ref.abs() + k * 2.0 ** -23 * mag + 1e-30
    assert bool((err <= bound * 1.0001).all()), f"max excess {float((err - bound).max())}"


def ref_mm(a, b, sa=1.0, sb=1.0, bias=None):
    r = (a.double() * sa) @ (b.double() * sb)
    mag = (a.double().abs() * abs(sa)) @ (b.double().abs() * abs(sb))
    if bias is not None:
        r = r + bias.double()
    return r, mag


@pytest.mark.parametrize("ta", [F8, F4, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("tb", [F8, F4, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("b_layout", ["row", "col"])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_matmul(ta, tb, b_layout, out_dtype):
    M, K, N = 70, 96, 50
    a = rand((M, K), ta, seed=1)
    b = rand((K, N), tb, seed=2) if b_layout == "row" else rand((N, K), tb, seed=2).t()
    y = fx().matmul(a, b, out_dtype=out_dtype)
    assert y.shape == (M, N) and y.dtype == out_dtype
    ref, mag = ref_mm(a, b)
    check_close(y, ref, mag, K, out_dtype)


@pytest.mark.parametrize("rows", [1, 3, 8, 9, 64])
@pytest.mark.parametrize("tx", [F8, F4, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("tw", [F8, F4])
def test_linear_fp8_weight(rows, tx, tw):
    N, K = 300, 512
    w = rand((N, K), tw, seed=3)
    x = rand((rows, K), tx, seed=4)
    bias = rand((N,), torch.bfloat16, seed=5)
    sw = torch.tensor([0.25], device=DEV)
    y = fx().linear(x, w, bias, scale_w=sw)
    ref, mag = ref_mm(x, w.t(), sb=0.25, bias=bias)
    check_close(y, ref, mag, K, torch.bfloat16)


def test_accumulate_fp32_out():
    M, K, N = 33, 64, 47
    a, b = rand((M, K), torch.bfloat16, seed=1), rand((K, N), torch.bfloat16, seed=2)
    out = rand((M, N), torch.float32, seed=3)
    ref = out.double() + a.double() @ b.double()
    mag = a.double().abs() @ b.double().abs() + out.double().abs()
    fx().matmul(a, b, out=out, beta=1.0)
    check_close(out, ref, mag, K, torch.float32)


def test_fp8_output_with_scale_and_amax():
    M, K, N = 64, 128, 48
    a, b = rand((M, K), F8, seed=1), rand((K, N), F4, seed=2)
    scale = torch.tensor([0.5], device=DEV)
    amax = torch.zeros(1, device=DEV)
    y = fx().matmul(a, b, out_dtype=F8, scale_out=scale, amax_out=amax)
    ref, mag = ref_mm(a, b)
    check_close(y.float() / 0.5, ref, mag / 1.0, K, F8)
    assert abs(float(amax) - float(ref.abs().max())) <= 1e-3 * float(ref.abs().max()) + K * 2.0 ** -23 * float(mag.max())


def test_rowwise_scales():
    M, K, N = 40, 64, 72
    a, b = rand((M, K), F8, seed=1), rand((K, N), F4, seed=2)
    sa = torch.rand(M, 1, device=DEV) + 0.5
    sb = torch.rand(1, N, device=DEV) + 0.5
    y = fx().matmul(a, b, out_dtype=torch.float32, scale_a=sa, scale_b=sb)
    ref = (a.double() * sa.double()) @ (b.double() * sb.double())
    mag = (a.double().abs() * sa.double()) @ (b.double().abs() * sb.double())
    check_close(y, ref, mag, K, torch.float32)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, F8, F4])
def test_cast_matches_torch_conversion_on_finite_values(dtype):
    x = rand((1000,), torch.float32, 3.0, seed=7)
    y = fx().cast(x, dtype)
    assert torch.equal(y.view(torch.uint8), x.to(dtype).view(torch.uint8))


def test_cast_known_answer():
    x = torch.tensor([1.0, float("inf"), -1e6, 3.0], device=DEV)
    amax = torch.zeros(1, device=DEV)
    y = fx().cast(x, F8, amax=amax)
    assert y.view(torch.uint8).tolist() == [0x3C, 0x7B, 0xFB, 0x42] and torch.isinf(amax).all()


def test_adamw_optimizer_tracks_torch():
    torch.manual_seed(0)
    w0 = torch.randn(257, 33, device=DEV)
    a = w0.clone().requires_grad_(True)
    b = w0.clone().requires_grad_(True)
    oa = torch.optim.AdamW([a], lr=1e-2, weight_decay=0.05)
    ob = fx().AdamW([b], lr=1e-2, weight_decay=0.05)
    for _ in range(5):
        g = torch.randn_like(w0)
        a.grad, b.grad = g.clone(), g.clone()
        oa.step(); ob.step()
    assert torch.allclose(a, b, rtol=2e-5, atol=2e-6)


def test_rejections():
    f = fx()
    a, b = rand((16, 32), F8), rand((32, 16), F8)
    with pytest.raises(ValueError, match="multiple of 16"):
        f.matmul(rand((16, 24), F8), rand((24, 16), F8))
    with pytest.raises(TypeError):
        f.matmul(a.to(torch.float16), b)
    with pytest.raises(ValueError, match="shapes"):
        f.matmul(a, rand((16, 16), F8))
    with pytest.raises(ValueError, match="scale_a"):
        f.matmul(a.to(torch.bfloat16), b, scale_a=torch.ones(1, device=DEV))
    with pytest.raises(ValueError, match="out must be given"):
        f.matmul(a, b, beta=1.0)
    with pytest.raises(ValueError, match="CUDA tensor"):
        f.cast(torch.zeros(4), F8)
    with pytest.raises(ValueError, match="step"):
        p = torch.zeros(8, device=DEV)
        f.adam_step(p, p.clone(), p.clone(), p.clone(), lr=1e-3, step=0)


def test_rejects_buffers_that_share_memory():
    """The reference binding refuses an output that overlaps an operand and optimizer arrays that overlap each
    other (binds/python/csrc/e5m2effma_torch.cpp:90,159-161,247-249)."""
    f = fx()
    x = torch.randn(16, 16, device=DEV)
    with pytest.raises(ValueError, match="share memory"):
        f.matmul(x, torch.randn(16, 16, device=DEV), out=x)
    with pytest.raises(ValueError, match="share memory"):
        f.matmul(torch.randn(16, 16, device=DEV), x.t(), out=x)
    p, g = torch.zeros(10, device=DEV), torch.zeros(10, device=DEV)
    m = torch.zeros(10, device=DEV)
    with pytest.raises(ValueError, match="share memory"):
        f.adam_step(p, g, m, m, lr=1e-3, step=1)
    with pytest.raises(ValueError, match="share memory"):
        f.adam_step(p, p, m, torch.zeros(10, device=DEV), lr=1e-3, step=1)
    with pytest.raises(ValueError, match="betas"):
        f.adam_step(p, g, m, torch.zeros(10, device=DEV), lr=1e-3, betas=(0.9, 1.0), step=1)
    with pytest.raises(ValueError):
        f.AdamW([torch.nn.Parameter(p)], lr=-1.0)


def test_optimizer_skips_empty_parameters():
    f = fx()
    w = torch.nn.Parameter(torch.randn(33, device=DEV))
    e = torch.nn.Parameter(torch.zeros(0, device=DEV))
    opt = f.AdamW([w, e], lr=1e-2)
    w.grad, e.grad = torch.randn(33, device=DEV), torch.zeros(0, device=DEV)
    before = w.detach().clone()
    opt.step()
    assert not torch.equal(before, w.detach())


def test_rejects_mixed_devices_and_runs_on_the_second_gpu():
    """binds/python/tests/test_e5m2effma.py:306-318."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    f = fx()
    a, b = rand((8, 16), F8), rand((16, 8), F8)
    with pytest.raises(ValueError, match="cuda:1"):
        f.matmul(a, b.to("cuda:1"))
    a1, b1 = a.to("cuda:1"), b.to("cuda:1")
    y = f.matmul(a1, b1)
    assert y.device == a1.device
    assert torch.equal(y.cpu(), f.matmul(a, b).cpu())
