"""Generates tests/golden/*.npz from the reference's own host code.

Run in a container that has the reference sources: `make -C oracle` compiles them (unchanged, from
where they lie) into oracle/_ref/libref.so (exact one-MAC model, tests/ref_capi.cpp) and
oracle/_ref/librefenc.so (host encoders src/e5m2effma.cuh:83-124 and element helpers
tests/test_util.h:21-56).  This script records their outputs on seeded inputs so that the pin
tests can run where the reference is absent.

    python tests/golden/make_golden.py
"""
import ctypes
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
E4M3, BF16, FP16, FP32, E5M2 = 0, 1, 2, 3, 4


def load_ref():
    enc = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "librefenc.so"))
    p, f = ctypes.c_void_p, ctypes.c_float
    enc.ref_hstore_n.argtypes = [ctypes.c_int, p, ctypes.c_size_t, p, f]
    enc.ref_hload_n.argtypes = [ctypes.c_int, p, ctypes.c_size_t, f, p]
    enc.ref_lane_n.argtypes = [ctypes.c_size_t, p, p, p, ctypes.c_int, ctypes.c_int, p]
    return enc


def ref_store(enc, dtype, values, qs, storage):
    v = np.ascontiguousarray(values, np.float32)
    out = np.zeros(v.size, storage)
    enc.ref_hstore_n(dtype, out.ctypes.data, v.size, v.ctypes.data, qs)
    return out


def ref_load(enc, dtype, raw, sinv):
    raw = np.ascontiguousarray(raw)
    out = np.zeros(raw.size, np.float32)
    enc.ref_hload_n(dtype, raw.ctypes.data, raw.size, sinv, out.ctypes.data)
    return out


def encoder_inputs(rng):
    """Bit patterns that stress the encoders: every FP8 value and midpoint of both formats with
    their FP32 neighbours, saturation thresholds, subnormal boundaries, specials, random bits."""
    pts = []
    for e in range(-30, 18):
        for frac in range(0, 64):
            pts.append(np.ldexp(1.0 + frac / 64.0, e))
    pts = np.array(pts, np.float32)
    u = pts.view(np.uint32)
    near = np.concatenate([u - 1, u, u + 1])
    special = np.array([0x00000000, 0x80000000, 0x7F800000, 0xFF800000, 0x7FC00000, 0xFFC00000, 0x7F800001,
                        0xFFFFFFFF, 0x00000001, 0x80000001, 0x007FFFFF, 0x00800000, 0x43E00000, 0x43DFFFFF,
                        0x43E00001, 0x47600000, 0x475FFFFF, 0x47600001, 0x477FF000, 0x477FEFFF, 0x33000000,
                        0x33000001, 0x32FFFFFF, 0x38800000, 0x387FFFFF, 0x3C800000, 0x3C7FFFFF], np.uint32)
    rnd = rng.integers(0, 2 ** 32, 60000, dtype=np.uint64).astype(np.uint32)
    bits = np.concatenate([near, near | 0x80000000, special, rnd])
    return bits.view(np.float32)


def main():
    enc = load_ref()
    rng = np.random.default_rng(20260101)
    x = encoder_inputs(rng)
    np.savez_compressed(
        os.path.join(HERE, "encoders.npz"), x_bits=x.view(np.uint32),
        e4m3=ref_store(enc, E4M3, x, 1.0, np.uint8), e5m2=ref_store(enc, E5M2, x, 1.0, np.uint8),
        bf16=ref_store(enc, BF16, x, 1.0, np.uint16), fp16=ref_store(enc, FP16, x, 1.0, np.uint16),
        e4m3_half=ref_store(enc, E4M3, x, 0.5, np.uint8), e5m2_half=ref_store(enc, E5M2, x, 0.5, np.uint8))

    codes = np.arange(256, dtype=np.uint8)
    h = rng.integers(0, 2 ** 16, 4096, dtype=np.uint64).astype(np.uint16)
    np.savez_compressed(
        os.path.join(HERE, "decoders.npz"), codes=codes, e4m3=ref_load(enc, E4M3, codes, 1.0).view(np.uint32),
        e5m2=ref_load(enc, E5M2, codes, 1.0).view(np.uint32),
        e4m3_half=ref_load(enc, E4M3, codes, 0.5).view(np.uint32),
        e5m2_half=ref_load(enc, E5M2, codes, 0.5).view(np.uint32),
        h_bits=h, bf16=ref_load(enc, BF16, h, 1.0).view(np.uint32), fp16=ref_load(enc, FP16, h, 1.0).view(np.uint32))

    out = {}
    for fa in (0, 1):
        for fb in (0, 1):
            n = 40000
            a = rng.integers(0, 256, n).astype(np.uint32)
            b = rng.integers(0, 256, n).astype(np.uint32)
            acc = rng.integers(0, 2 ** 16, n).astype(np.uint32)
            # near cancellation: accumulator = minus the rounded product, perturbed by a few BF16 ulps
            fin_a = np.where(fa == 1, (a & 0x7C) != 0x7C, (a & 0x7F) != 0x7F)
            fin_b = np.where(fb == 1, (b & 0x7C) != 0x7C, (b & 0x7F) != 0x7F)
            va = ref_load(enc, E5M2 if fa else E4M3, a.astype(np.uint8), 1.0).astype(np.float64)
            vb = ref_load(enc, E5M2 if fb else E4M3, b.astype(np.uint8), 1.0).astype(np.float64)
            prod = np.where(fin_a & fin_b, -(va * vb), 0.0).astype(np.float32)
            pb = (prod.view(np.uint32) >> 16).astype(np.int64) + rng.integers(-2, 3, n)
            half = n // 2
            acc[:half] = (pb[:half] & 0xFFFF).astype(np.uint32)
            res = np.zeros(n, np.uint32)
            enc.ref_lane_n(n, a.ctypes.data, b.ctypes.data, acc.ctypes.data, fa, fb, res.ctypes.data)
            out[f"a_{fa}{fb}"] = a.astype(np.uint8)
            out[f"b_{fa}{fb}"] = b.astype(np.uint8)
            out[f"acc_{fa}{fb}"] = acc.astype(np.uint16)
            out[f"res_{fa}{fb}"] = res.astype(np.uint16)
    np.savez_compressed(os.path.join(HERE, "lane.npz"), **out)
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()
