"""Properties of the oracle's codecs and an independent cross-check (CPU only).

The pins in test_oracle_pins.py tie the oracle to the reference's own encoders.  These tests add what a
codec must satisfy by construction -- decode/encode round trips over every code, monotonicity, ties to even,
saturation -- and compare with PyTorch's CPU conversions (an implementation that shares no code with either)
wherever the two conventions coincide: every finite in-range value for FP8, every non-NaN value for BF16 / FP16."""
import numpy as np
import pytest
import torch

import oracle as orc

FP8 = [(orc.E5M2, torch.float8_e5m2, 57344.0), (orc.E4M3, torch.float8_e4m3fn, 448.0)]


def finite_codes(dtype):
    c = np.arange(256, dtype=np.uint8)
    if dtype == orc.E5M2:
        return c[(c & 0x7C) != 0x7C]
    return c[(c & 0x7F) != 0x7F]


@pytest.mark.parametrize("dtype,tdt,fmax", FP8)
def test_every_finite_code_round_trips(dtype, tdt, fmax):
    c = finite_codes(dtype)
    v = orc.decode(dtype, c)
    back = orc.encode(dtype, v)
    # -0 and +0 keep their sign; every other code is the unique representation of its value
    assert np.array_equal(back, c)
    assert float(np.abs(v).max()) == fmax


@pytest.mark.parametrize("dtype,tdt,fmax", FP8)
def test_decode_agrees_with_torch_on_every_finite_code(dtype, tdt, fmax):
    c = finite_codes(dtype)
    ours = orc.decode(dtype, c)
    theirs = torch.from_numpy(c.copy()).view(tdt).to(torch.float32).numpy()
    assert np.array_equal(ours.view(np.uint32), theirs.view(np.uint32))


@pytest.mark.parametrize("dtype,tdt,fmax", FP8)
def test_encode_agrees_with_torch_inside_the_finite_range(dtype, tdt, fmax):
    rng = np.random.default_rng(11)
    bits = rng.integers(0, 2 ** 32, 2_000_000, dtype=np.uint64).astype(np.uint32)
    x = bits.view(np.float32)
    x = x[np.isfinite(x) & (np.abs(x) <= fmax)]
    # plus values that sit exactly on, and one float next to, every rounding boundary
    grid = np.sort(np.unique(np.abs(orc.decode(dtype, finite_codes(dtype)))))
    mid = ((grid[:-1].astype(np.float64) + grid[1:].astype(np.float64)) / 2).astype(np.float32)
    edge = np.concatenate([mid, np.nextafter(mid, np.float32(0)), np.nextafter(mid, np.float32(np.inf)), grid])
    x = np.concatenate([x, edge, -edge]).astype(np.float32)
    ours = orc.encode(dtype, x)
    theirs = torch.from_numpy(x.copy()).to(tdt).view(torch.uint8).numpy()
    assert np.array_equal(ours, theirs)


@pytest.mark.parametrize("dtype,tdt,fmax", FP8)
def test_encode_is_monotonic_and_saturates(dtype, tdt, fmax):
    rng = np.random.default_rng(12)
    x = np.sort(np.concatenate([rng.standard_normal(200_000).astype(np.float32) * s for s in (1e-6, 1e-2, 1.0, 300.0, 1e6)]))
    v = orc.decode(dtype, orc.encode(dtype, x))
    assert np.all(np.diff(v) >= 0)
    top = orc.encode(dtype, np.array([fmax * 4, np.inf, -fmax * 4, -np.inf], np.float32))
    expect = (0x7B, 0x7B, 0xFB, 0xFB) if dtype == orc.E5M2 else (0x7E, 0x7E, 0xFE, 0xFE)
    assert tuple(int(t) for t in top) == expect
    nan = np.array([np.nan, -np.nan], np.float32)
    assert [int(t) for t in orc.encode(dtype, nan)] == [0x7F, 0x7F]


@pytest.mark.parametrize("dtype,tdt", [(orc.BF16, torch.bfloat16), (orc.FP16, torch.float16)])
def test_16_bit_encoders_agree_with_torch_on_every_non_nan_value(dtype, tdt):
    rng = np.random.default_rng(13)
    bits = rng.integers(0, 2 ** 32, 3_000_000, dtype=np.uint64).astype(np.uint32)
    # every exponent, and the 2^16 patterns around each tie of the discarded half for BF16
    ties = (np.arange(1 << 16, dtype=np.uint32) << 16)[:, None] + np.array([0x7FFF, 0x8000, 0x8001], np.uint32)[None, :]
    x = np.concatenate([bits, ties.reshape(-1)]).view(np.float32)
    x = x[~np.isnan(x)]
    ours = orc.encode(dtype, x)
    theirs = torch.from_numpy(x.copy()).to(tdt).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(ours, theirs)
    back = orc.decode(dtype, ours)
    assert np.array_equal(back.view(np.uint32), torch.from_numpy(theirs.view(np.int16).copy()).view(tdt).to(torch.float32).numpy().view(np.uint32))


def test_nan_conventions_of_the_16_bit_encoders():
    nan = np.array([np.nan, -np.nan], np.float32)
    assert [int(t) for t in orc.encode(orc.BF16, nan)] == [0x7FC0, 0x7FC0]
    assert [int(t) for t in orc.encode(orc.FP16, nan)] == [0x7FFF, 0x7FFF]


@pytest.mark.parametrize("adamw", [1, 0])
def test_adam_follows_the_textbook_update(adamw):
    """Three FP32 steps of the oracle against torch.optim.AdamW / Adam on the CPU.  The two order their FP32
    operations differently, so agreement is to a few ulp, not bit for bit: this guards the formula (bias
    corrections, decoupled against L2 weight decay, eps outside the square root), not the rounding."""
    rng = np.random.default_rng(21)
    n = 4096
    p0 = (rng.standard_normal(n) * 0.05).astype(np.float32)
    hp = dict(lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1)
    p, m, v = p0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
    tp = torch.nn.Parameter(torch.from_numpy(p0.copy()))
    cls = torch.optim.AdamW if adamw else torch.optim.Adam
    opt = cls([tp], lr=hp["lr"], betas=(hp["beta1"], hp["beta2"]), eps=hp["eps"], weight_decay=hp["weight_decay"])
    for step in (1, 2, 3):
        g = (rng.standard_normal(n) * 1e-2).astype(np.float32)
        orc.adam(dict(hp, step=step, adamw=adamw, bias_correction=1, grad_scale=1.0), p, orc.FP32, g, orc.FP32, m, v, orc.FP32)
        tp.grad = torch.from_numpy(g.copy())
        opt.step()
    np.testing.assert_allclose(p, tp.detach().numpy(), rtol=2e-5, atol=1e-8)
