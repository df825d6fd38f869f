"""Kernel-selection sweep for one GPU: times the alternatives the library can be steered to through its
experiment switches and prints which one wins per shape -- the role `make tune` (tune/tune.cu:52-118)
plays for the reference.  The library's built-in choices were set from this sweep on a B200; run it on
another sm_100 part to check that they still hold.

    python -m e5m2effma_b200.tune            # GEMM pair / single CTA, tail slicing, GEMV variants
"""
import os
import sys

import torch

from . import capi, workloads

SWITCHES = {
    "gemm": [("pair + tail slices", {"E5MA_TC_PAIR": "1", "E5MA_TC_SPLIT": "1"}),
             ("pair", {"E5MA_TC_PAIR": "1", "E5MA_TC_SPLIT": "0"}),
             ("single CTA + half tiles", {"E5MA_TC_PAIR": "0", "E5MA_TC_SPLIT": "1"}),
             ("single CTA", {"E5MA_TC_PAIR": "0", "E5MA_TC_SPLIT": "0"})],
    "gemv": [("cp.async, 2 stages", {"E5MA_GEMV_ASYNC": "1", "E5MA_GEMV_STAGES": "2"}),
             ("cp.async, 3 stages", {"E5MA_GEMV_ASYNC": "1", "E5MA_GEMV_STAGES": "3"}),
             ("register loads", {"E5MA_GEMV_ASYNC": "0"})],
}


def time_us(w, steps=20, rot_bytes=260e6):
    """Average time of one pass in microseconds: `steps` launches over rotating operand copies larger
    than L2, replayed as one CUDA graph, timed with CUDA events."""
    s = torch.cuda.current_stream()
    per = w.A.numel() * w.A.element_size() + w.B.numel() * w.B.element_size()
    sets = max(1, int(rot_bytes // per) + 1) if per < 200e6 else 1
    rot = [(w.A.clone(), w.B.clone()) for _ in range(sets)]
    for i in range(3):
        w.launch(s.cuda_stream, *rot[i % sets])
    torch.cuda.synchronize()
    cs = torch.cuda.Stream()
    cs.wait_stream(s)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(cs):
        with torch.cuda.graph(g, stream=cs):
            for i in range(steps):
                w.launch(cs.cuda_stream, *rot[i % sets])
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps * 1e3


def main():
    dev = torch.device("cuda", 0)
    shapes = [("gemm", 4096, 4096, 4096), ("gemm", 8192, 4096, 14336), ("gemm", 2048, 2048, 2048), ("gemm", 1024, 8192, 4096),
              ("gemv", 8192, 1, 8192), ("gemv", 8192, 8, 8192), ("gemv", 4096, 4, 14336)]
    saved = {k: os.environ.get(k) for _, alts in SWITCHES.items() for _, env in alts for k in env}
    for kind, m, n, k in shapes:
        if kind == "gemm":
            w = workloads.GemmWorkload("tune", m, n, k, capi.E5M2, capi.E5M2, capi.BF16, dev, a_std=8.0, b_std=8.0,
                                       a_scale_inv=0.125, b_scale_inv=0.125, seed=1)
        else:
            w = workloads.GemmWorkload("tune", m, n, k, capi.E5M2, capi.BF16, capi.BF16, dev, a_std=0.02, a_scaling="outer", seed=2)
        rows = []
        for label, env in SWITCHES[kind]:
            for key in saved:
                os.environ.pop(key, None)
            os.environ.update(env)
            rows.append((time_us(w), label))
        best = min(rows)
        print(f"{kind} m={m} n={n} k={k}: " + "; ".join(f"{lbl} {us:.1f} us" for us, lbl in rows) + f"  -> {best[1]}", flush=True)
        del w
        torch.cuda.empty_cache()
    for key, val in saved.items():
        os.environ.pop(key, None)
        if val is not None:
            os.environ[key] = val
    if capi.gemm_fault():
        print("a bounded wait ran out during the sweep (see e5b_gemm_fault)", file=sys.stderr)


if __name__ == "__main__":
    main()
