#!/usr/bin/env python
"""Benchmark of the hot path through the C interface.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One "step" is one pass of the chosen workload (default: c2, the HYBRID dgrad GEMM 8192 x 4096 x 14336,
E5M2 row-wise x E4M3 + BF16 bias -> E5M2 + amax) over synthetic, seeded inputs.  One JSON line goes to stdout:

  value      whole-job throughput with the inputs resident in HBM (TFLOP/s for GEMMs, GB/s for the
             bandwidth-bound workloads), timed with CUDA events on the launching stream over exactly K steps,
             max over ranks
  e2e        the same metric with the step's inputs starting in pinned host memory: host-to-device copies, the
             call through the C interface and the device-to-host read of the result are all inside the timed region
  roofline   algorithmic FLOPs (or bytes) per launch / average launch time, against the measured peak of
             MEASURED_PEAKS.json (FP8: twice the measured BF16 figure); .sustained is the same kernel looped for
             seconds, until the power-capped clocks have settled, against the sustained peak
  workloads  after the headline, the other configurations of the metric (c1, c3n1, c3n8, c4, c5, one cast) with
             the same protocol: time, value, roofline, clocks
  gemm_rows  (N = 1) the rows of the reference's own GEMM benchmark at M = N = K = 4096: the four operand layouts
             TN / NN / NT / TT, the E5M2 x E4M3, E5M2 x BF16 and E5M2 x FP32 pairings and the FP32 accumulate mode,
             then those of its GEMV benchmark (x in E5M2 / BF16 / FP32, batch 1, 2, 4, 8), each with the kernel that took it
  cpu_baseline  the CPU oracle (a restatement of the reference's host emulation) on a bounded column slab of the
             very operands the GPU just used, all host threads (rank 0, N = 1 only); .observed_error is the
             largest difference between the GPU result and the oracle's double-precision value, in units of
             2^-23 * sum|a*b|*|s| (an "effective k"; the stated bound allows k) and in ulps of the output format

N > 1 (torchrun, one rank per GPU): the stated problem is SHARDED, its total size fixed ("strong" scaling): GEMMs
by column blocks of B / D with A replicated, the GEMV by weight rows, AdamW / casts by element chunks.  The step
then contains the collectives the sharding needs: the all-gather of the output blocks -- fused into the GEMM /
GEMV epilogue, which stores its block straight into every peer's copy of D over NVLink (e5b_gemm_bcast); the same
step with an NCCL all-gather after a plain e5ma_gemm is timed beside it -- and the max-all-reduce of the scalar
amax.  weak_scaling keeps the weak-scaling figure (every rank the full problem, amax reduction only).

--impl reference times the reference's own CPU algorithm (the oracle port: the reference's GPU kernels refuse
this architecture and its host emulation does not build stand-alone) on the same seeded inputs and prints the
same line with "impl": "reference".
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# DRAM traffic per launch (dram__bytes_read.sum + dram__bytes_write.sum) from one ncu capture per kernel and
# workload (the summaries are committed); None where no capture has been taken.  Shrunk captures are scaled
# linearly to the full element count (AdamW, casts: traffic is proportional to the count).
NCU_TRAFFIC_BYTES = {
    "c2": 368.6e6, "c1": 34.5e6, "c4": 2173.5e6, "c3n1": 68.8e6, "c3n8": 67.8e6, "c5": 15.67e9, "cast_e4m3_bf16": 2.987e9,
}

GEMM_LIKE = ("c1", "c2", "c4")
EXTRAS = ["c1", "c3n1", "c3n8", "c4", "c5", "cast_e4m3_bf16"]
METRIC = {"c1": "fp8_gemm_4096_e5m2_bf16", "c2": "fp8_hybrid_dgrad_gemm", "c4": "wgrad_e5m2_bf16_fp32_accumulate",
          "c3n1": "gemv_8192_e5m2_bf16_batch1", "c3n8": "gemv_8192_e5m2_bf16_batch8", "c5": "fused_adamw_bf16_e4m3_copy"}
DESC = {"c1": "GEMM M=N=K=4096 E5M2 x E5M2 (TN, scale_inv 0.125) -> BF16",
        "c2": "HYBRID dgrad GEMM M=8192 N=4096 K=14336, E5M2 row-wise x E4M3 per-tensor + BF16 bias -> E5M2 + amax",
        "c3n1": "decode GEMV W 8192x8192 E5M2 row-wise, x BF16 batch 1 -> BF16",
        "c3n8": "decode GEMV W 8192x8192 E5M2 row-wise, x BF16 batch 8 -> BF16",
        "c4": "wgrad GEMM M=N=4096 K=65536 E5M2 x BF16, beta=1 into FP32 main_grad",
        "c5": "fused AdamW over 2^30 BF16 parameters, BF16 m/v, E4M3 copy + amax"}
DTYPE = {"c1": "fp8 (e5m2 x e5m2, f32 accumulate)", "c2": "fp8 (e5m2 x e4m3, f32 accumulate)",
         "c4": "bf16 (e5m2 widened exactly, f32 accumulate)"}
TOLERANCE = ("GEMM/GEMV: 1 ulp of the output format + k * 2^-23 * sum|a*b|*|s| (checked by tests/ on every output of the small "
             "cases and on sampled rows/columns at full size); casts, AdamW: bit-exact")


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "bf16_tflops_sustained": p.get("bf16_tflops_sustained"),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while a timed region runs (read-only)."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.stop_flag, self.max_mhz = index, [], set(), False, None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def sample(self):
        if self.nv is None:
            return
        nv = self.nv
        names = {nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
                 nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
                 nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
                 nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap"}
        try:
            self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
            r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
            for bit, nm in names.items():
                if r & bit:
                    self.reasons.add(nm)
        except Exception:
            pass

    def run(self):
        while not self.stop_flag:
            self.sample()
            time.sleep(0.005)

    def poll_until(self, event):
        """Samples from the calling thread while the GPU works through what has already been enqueued, until
        `event` has completed (a sampling thread beside the launching thread delays launches now and then, and with a
        collective in every step all ranks pay for each such delay)."""
        self.sample()
        while not event.query():
            self.sample()
            time.sleep(0.0005)

    def reset(self):
        self.samples, self.reasons = [], set()

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


# ---------------------------------------------------------------------------------------------------------------
# CPU arm: the oracle on the very operands of a workload
# ---------------------------------------------------------------------------------------------------------------
NP_OF = None


def _np_storage():
    global NP_OF
    if NP_OF is None:
        import numpy as np
        NP_OF = {0: np.uint8, 4: np.uint8, 1: np.uint16, 2: np.uint16, 3: np.float32}
    return NP_OF


def host(t, dtype_code=None):
    """A torch tensor's raw storage as a flat numpy array of the oracle's storage type."""
    import torch
    raw = t.detach().cpu().contiguous().view(torch.uint8).numpy()
    return raw if dtype_code is None else raw.view(_np_storage()[dtype_code]).reshape(-1)


class HostGemm:
    """Host copies of a GEMM workload's operands, made once."""

    def __init__(self, w, d_dtype=None, d_scale=None):
        self.w = w
        self.A, self.B = host(w.A, w.a_dtype), host(w.B, w.b_dtype)
        self.sa = None if w.sa is None else w.sa.cpu().numpy()
        self.sb = None if w.sb is None else w.sb.cpu().numpy()
        self.bias = None if w.bias is None else host(w.bias, 1)
        self.C0 = None if w.D0 is None else host(w.D0, w.d_dtype)
        self.d_dtype = w.d_dtype if d_dtype is None else d_dtype
        ds = w.d_scale if d_scale is None else d_scale
        self.d_scale = None if ds is None else (float(ds.item()) if hasattr(ds, "item") else float(ds))

    def wide(self, orc, cols):
        w = self.w
        return orc.gemm_wide(1, 0, w.m, w.n, w.k, 1.0, self.A, w.a_dtype, w.k, self.B, w.b_dtype, w.k, w.beta, self.C0,
                             self.d_dtype, w.m, bias=self.bias, bias_dtype=orc.BF16, a_sinv=self.sa, a_outer=w.a_outer,
                             b_sinv=self.sb, b_outer=w.b_outer, cols=cols)

    def timed_slab(self, orc, cols):
        """The reference-order GEMM (ascending-k FP32 chain, full epilogue, conversion, amax) on output columns
        [cols[0], cols[1]); returns (seconds, amax)."""
        import numpy as np
        w = self.w
        D = np.zeros(w.n * w.m, _np_storage()[self.d_dtype]) if self.C0 is None or self.d_dtype != w.d_dtype else self.C0.copy()
        t = time.perf_counter()
        am = orc.gemm(1, 0, w.m, w.n, w.k, 1.0, self.A, w.a_dtype, w.k, self.B, w.b_dtype, w.k, w.beta,
                      self.C0 if w.beta != 0.0 else None, self.d_dtype, w.m, D, self.d_dtype, w.m, bias=self.bias,
                      bias_dtype=orc.BF16, a_sinv=self.sa, a_outer=w.a_outer, b_sinv=self.sb, b_outer=w.b_outer,
                      d_scale=self.d_scale if self.d_dtype in (0, 4) else None, amax=0.0 if w.amax is not None else None, cols=cols)
        return time.perf_counter() - t, am


def cpu_gemm(w, orc, target_s, d_dtype=None, d_scale=None, hg=None):
    """(value, unit, sample description, seconds) of the oracle on a bounded column slab of workload w's own operands."""
    hg = hg or HostGemm(w, d_dtype, d_scale)
    cols = w.n
    if w.n > 8:
        # calibrate the slab width on growing probes (a narrow probe underuses the threads and would mislead)
        probe = min(w.n, 4 * orc.threads())
        while True:
            t0, _ = hg.timed_slab(orc, (0, probe))
            if t0 >= 0.5 or probe >= w.n:
                break
            probe = min(w.n, probe * 4)
        cols = int(max(probe, min(w.n, probe * target_s / max(t0, 1e-9)))) // 4 * 4
    t1, _ = hg.timed_slab(orc, (0, cols))
    what = f"all {w.m} rows, first {cols} of {w.n} output columns, full k = {w.k}, the GPU arm's own operands, scales and bias: {t1:.2f} s"
    if w.unit_name == "B":
        return (float(w.m) * w.k + 2.0 * w.k * cols + 4.0 * w.m + 2.0 * w.m * cols) / t1 / 1e9, "GB/s", what, t1
    return 2.0 * w.m * cols * w.k / t1 / 1e12, "TFLOP/s", what, t1


def cpu_adam(w, orc, count=1 << 26):
    count = min(count, w.count)
    p, g = host(w.p[:count], 1).copy(), host(w.g[:count], 1).copy()
    import numpy as np
    mm, vv, q = np.zeros(count, np.uint16), np.zeros(count, np.uint16), np.zeros(count, np.uint8)
    cfg = dict(lr=3e-4, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.1, step=1, adamw=1, bias_correction=1, grad_scale=1.0)
    t = time.perf_counter()
    orc.adam(cfg, p, orc.BF16, g, orc.BF16, mm, vv, orc.BF16, q, orc.E4M3, 2048.0, 0.0)
    t1 = time.perf_counter() - t
    return count * 15.0 / t1 / 1e9, "GB/s", f"the first {count} of {w.count} parameters (same seeded p and g): {t1:.2f} s", t1


def cpu_cast(w, orc, count=1 << 27):
    es = {3: 4, 1: 2, 2: 2, 0: 1, 4: 1}
    count = min(count, w.count)
    src = host(w.src[:count], w.src_dtype).copy()
    t = time.perf_counter()
    orc.cast(src, w.src_dtype, w.dst_dtype, 16.0 if w.src_dtype in (0, 4) else None, 16.0 if w.dst_dtype in (0, 4) else None, amax=0.0)
    t1 = time.perf_counter() - t
    return count * (es[w.src_dtype] + es[w.dst_dtype]) / t1 / 1e9, "GB/s", f"the first {count} of {w.count} elements: {t1:.2f} s", t1


def cpu_sample(w, orc, target_s, **kw):
    if w.kind == "gemm":
        return cpu_gemm(w, orc, target_s, **kw)
    if w.kind == "adam":
        return cpu_adam(w, orc)
    return cpu_cast(w, orc)


def observed_error(hg, orc, D_cols, cols, out_dtype):
    """Largest deviation of the GPU's output columns from the oracle's double-precision value: in units of
    2^-23 * sum|a*b|*|s| (how many FP32 roundings of the magnitude sum it corresponds to; the stated bound allows k of
    them on top of one output ulp) and in ulps of the output format at the reference value.  Nothing is subtracted."""
    import numpy as np
    mant = {1: 8, 2: 11, 3: 24}[out_dtype]
    worst_k, worst_ulp, inside = 0.0, 0.0, True
    for (j0, j1), got_raw in zip(cols, D_cols):
        ref, mag, fix = hg.wide(orc, (j0, j1))
        got = orc.decode(out_dtype, got_raw.reshape(-1), 1.0).astype(np.float64).reshape(ref.shape)
        err = np.abs(got - ref)
        ulp = np.exp2(np.floor(np.log2(np.maximum(np.abs(ref), 1e-300))) - (mant - 1))
        worst_k = max(worst_k, float((err / np.maximum(2.0 ** -23 * mag, 1e-300)).max()))
        worst_ulp = max(worst_ulp, float((err / ulp).max()))
        inside = inside and bool((err <= ulp + hg.w.k * 2.0 ** -23 * mag + 2.0 ** -21 * (np.abs(ref) + fix + mag)).all())
    rep = {"columns": sum(b - a for a, b in cols), "rows": int(hg.w.m), "output": {1: "BF16", 2: "FP16", 3: "FP32"}[out_dtype],
           "bound": f"1 output ulp + k * 2^-23 * sum|a*b|*|s| with k = {hg.w.k}", "inside_bound": inside}
    if out_dtype == 3:      # FP32 output: the summation error shows; an "effective k" (the bound allows k of these units)
        rep["max_error_in_units_of_2^-23_sum_abs_products"] = worst_k
    else:                   # 16-bit output: its own rounding (up to 0.5 ulp) dominates
        rep["max_error_in_output_ulps"] = worst_ulp
    return rep


def error_report(w, orc, cols, first_pass=None):
    """Observed error of GEMM workload w on the given output columns, from fresh launches on its original operands:
    "accumulation" from a launch with FP32 output (nothing but the tensor core's summation and the epilogue's few
    FP32 operations separate it from the exact value), "output" from the configured output dtype when that is a
    16-bit format (or from first_pass: host copies of those columns from an earlier BF16 launch)."""
    import torch
    from e5m2effma_b200 import capi
    stream = torch.cuda.current_stream().cuda_stream
    saved = (w.d_dtype, w.D, w.d_scale, w.amax)
    rep = {}
    try:
        w.d_dtype, w.d_scale, w.amax = capi.FP32, None, None
        w.D = w.D0.clone() if (w.D0 is not None and saved[0] == capi.FP32) else torch.zeros((w.n, w.m), dtype=torch.float32, device=w.dev)
        if w.beta != 0.0 and saved[0] != capi.FP32:
            return {"skipped": "accumulating workload with a non-FP32 D"}
        w.launch(stream)
        torch.cuda.synchronize()
        got = [host(w.D[j0:j1], capi.FP32).copy() for j0, j1 in cols]
        rep["accumulation"] = observed_error(HostGemm(w), orc, got, cols, capi.FP32)
    finally:
        w.d_dtype, w.D, w.d_scale, w.amax = saved
    out_dt = capi.BF16 if first_pass is not None else w.d_dtype
    if out_dt in (capi.BF16, capi.FP16):
        if first_pass is None:
            w.launch(stream)
            torch.cuda.synchronize()
            first_pass = [host(w.D[j0:j1], out_dt).copy() for j0, j1 in cols]
        rep["output"] = observed_error(HostGemm(w, d_dtype=out_dt), orc, first_pass, cols, out_dt)
    return rep


# ---------------------------------------------------------------------------------------------------------------
# workloads on the GPU
# ---------------------------------------------------------------------------------------------------------------
def build_workload(name, dev, shrink, world=1, keep_first_pass=None):
    """The named workload on `dev`.  c2 needs prev_amax: a first pass of the same operands with BF16 output supplies
    it (max-reduced over the ranks; every rank holds the same full problem).  keep_first_pass: column ranges of that
    BF16 result to keep on the host for the error report."""
    import torch
    import torch.distributed as dist
    from e5m2effma_b200 import capi, workloads
    if name != "c2":
        return workloads.make(name, dev, shrink), None
    first = workloads.make("c2_bf16", dev, shrink)
    first.launch(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    kept = None
    if keep_first_pass:
        kept = [host(first.D[j0:j1], 1).copy() for j0, j1 in keep_first_pass]
    t = first.amax.clone()
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    prev_amax = float(t.item())
    w = first
    w.name = "c2"
    w.d_dtype = capi.E5M2
    w.D = torch.zeros((w.n, w.m), dtype=torch.uint8, device=dev)
    workloads.finish_c2(w, prev_amax)
    return w, kept


def rotation(w, world=1, extra_bytes=260e6):
    """Operand sets that together exceed L2 for workloads whose operands alone would fit (c1, c3): as many copies
    as it takes for the bytes ONE RANK touches per pass (its shard when the problem is sharded) to add up to more
    than L2 over one rotation."""
    if w.kind != "gemm":
        return None
    a, b = w.A.numel() * w.A.element_size(), w.B.numel() * w.B.element_size()
    per = (a / world + b) if w.n <= 8 else (a + b / world)
    if per >= 200e6:
        return None
    return [(w.A.clone(), w.B.clone()) for _ in range(min(48, int(extra_bytes // per) + 1))]


def make_step(w, rot):
    def step(i, sptr):
        if rot is not None:
            a, b = rot[i % len(rot)]
            w.launch(sptr, a, b)
        else:
            w.launch(sptr)
    return step


class Timing:
    """K steps on the GPU between two events; barrier + synchronize on both sides; max over ranks."""

    def __init__(self, dev, world):
        import torch
        self.torch, self.dev, self.world = torch, dev, world
        self.stream = torch.cuda.current_stream()

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, ms):
        if self.world > 1:
            import torch.distributed as dist
            t = self.torch.tensor([ms], device=self.dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def run(self, step, steps, warmup, graph, sampler=None, graph_optional=False, min_ms=0.0):
        """step(i, stream_ptr).  graph=True: the K steps are captured once into a CUDA graph and replayed (so that
        microsecond-scale kernels are not timed behind the Python launch path); steps with NCCL calls run on the stream.
        min_ms > 0: a graph whose K steps take less than that is replayed several times back to back inside the timed
        region (the same number of times on every rank) -- with steps that wait for other ranks, the few hundred
        microseconds by which the ranks' host threads start their replays apart would otherwise be what is timed."""
        torch, stream = self.torch, self.stream
        # W warm-up steps, and more of them until about 10 ms of GPU work have run: after an idle spell the SM clock
        # needs milliseconds to come back up, which a handful of microsecond-scale launches would not cover
        w0, w1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        w0.record(stream)
        for i in range(warmup):
            step(i, stream.cuda_stream)
        w1.record(stream)
        self.barrier()
        per = self.max_over_ranks(w0.elapsed_time(w1)) / max(warmup, 1)
        for i in range(min(2000, int(10.0 / max(per, 1e-3)) - warmup)):
            step(warmup + i, stream.cuda_stream)
        self.barrier()
        g = None
        if graph:
            try:
                cs = torch.cuda.Stream()
                cs.wait_stream(stream)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.stream(cs):
                    with torch.cuda.graph(g, stream=cs):
                        for i in range(steps):
                            step(i, cs.cuda_stream)
                g.replay()
            except Exception:
                if not graph_optional:
                    raise
                g = None
            self.barrier()
        self.timed_as = "cuda_graph" if g is not None else "stream"
        reps = 1
        if g is not None and min_ms > 0:
            p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            p0.record(stream)
            g.replay()
            p1.record(stream)
            self.barrier()
            reps = max(1, min(64, int(min_ms / max(self.max_over_ranks(p0.elapsed_time(p1)), 1e-3)) + 1))
        self.replays = reps
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        if g is not None:
            for _ in range(reps):
                g.replay()
        else:
            for i in range(steps):
                step(i, stream.cuda_stream)
        e1.record(stream)
        if sampler is not None:
            sampler.poll_until(e1)
        self.barrier()
        return self.max_over_ranks(e0.elapsed_time(e1)) / (steps * reps)

    def sustained(self, step, est_ms, sampler, seconds=2.0):
        """The same step looped for `seconds`: graph replays of ~30 ms each, NVML sampled from this thread between
        them; the figure is taken over the second half, when the power-capped clocks have settled."""
        torch, stream = self.torch, self.stream
        per = max(1, int(30.0 / max(est_ms, 1e-3)))
        cs = torch.cuda.Stream()
        cs.wait_stream(stream)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(cs):
            with torch.cuda.graph(g, stream=cs):
                for i in range(per):
                    step(i, cs.cuda_stream)
        replays = max(4, int(seconds * 1e3 / (per * est_ms)))
        half = replays // 2
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sampler.reset()
        for r in range(replays):
            if r == half:
                e0.record(stream)
                sampler.reset()
            g.replay()
            sampler.sample()
        e1.record(stream)
        sampler.poll_until(e1)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / ((replays - half) * per)
        return ms, sampler.summary(), replays * per


def roofline(name, w, ms_per_step, pk, units=None):
    units = w.units if units is None else units
    if name in GEMM_LIKE:
        fp8 = name != "c4"
        peak = pk["bf16_tflops"] * (2.0 if fp8 else 1.0)
        roof = {"bound": "tensor", "achieved": units / (ms_per_step * 1e-3) / 1e12, "peak": peak, "unit": "TFLOP/s",
                "peak_source": f"{pk['source']}: " + ("2 x bf16_tflops burst (FP8 issues at twice the BF16 rate)" if fp8 else "bf16_tflops burst"),
                "nominal_peak": 4500.0 if fp8 else 2250.0}
    else:
        roof = {"bound": "hbm", "achieved": units / (ms_per_step * 1e-3) / 1e9, "peak": pk["hbm_gbs"], "unit": "GB/s",
                "peak_source": f"{pk['source']}: hbm_gbs (copy)", "nominal_peak": 8000.0}
    roof["frac"] = roof["achieved"] / roof["peak"]
    roof["frac_of_nominal"] = roof["achieved"] / roof["nominal_peak"]
    roof["traffic"] = NCU_TRAFFIC_BYTES.get(name)
    roof["algorithmic_units_per_launch"] = units
    roof["kernel_ms"] = ms_per_step
    return roof


def sustained_entry(name, w, ms, clocks, launches, pk):
    fp8 = name in GEMM_LIKE and name != "c4"
    ach = w.units / (ms * 1e-3) / (1e12 if name in GEMM_LIKE else 1e9)
    if name in GEMM_LIKE:
        peak = (pk["bf16_tflops_sustained"] or pk["bf16_tflops"]) * (2.0 if fp8 else 1.0)
        src = f"{pk['source']}: " + ("2 x " if fp8 else "") + "bf16_tflops_sustained"
        nominal = 4500.0 if fp8 else 2250.0
    else:
        peak, src, nominal = pk["hbm_gbs"], f"{pk['source']}: hbm_gbs (copy)", 8000.0
    mhz = clocks.get("sm_mhz")
    return {"ms_per_step": ms, "achieved": ach, "peak": peak, "peak_source": src, "frac": ach / peak, "frac_of_nominal": ach / nominal,
            "launches": launches, "clocks": clocks, "ms_times_mhz": (ms * mhz if mhz else None),
            "note": "the same launch repeated for about two seconds; timed over the second half, NVML sampled between graph replays"}


# ---------------------------------------------------------------------------------------------------------------
# N > 1: the stated problem sharded over the ranks
# ---------------------------------------------------------------------------------------------------------------
class Sharded:
    """One rank's share of a workload through the unchanged C interface, and the collectives its output needs."""

    def __init__(self, name, w, world, rank, dev, rot=None, use_peers=True):
        import torch
        import torch.distributed as dist
        from e5m2effma_b200 import capi, sharding
        self.torch, self.dist, self.capi = torch, dist, capi
        self.name, self.w, self.world, self.rank = name, w, world, rank
        self.peerbuf, self.peer_note = None, None
        self.gather_bytes = 0
        if w.kind == "gemm":
            es = w.D.element_size()
            self.needs_gather = name != "c4"             # main_grad stays sharded
            if use_peers and self.needs_gather:
                try:
                    from e5m2effma_b200.peer import PeerBuffer
                    self.peerbuf = PeerBuffer(w.D.numel() * es, dev)
                    w.D = self.peerbuf.local[: w.D.numel() * es].view(w.D.dtype).view(w.D.shape)
                except Exception as e:                   # no peer mapping on this system: NCCL all-gather only
                    self.peer_note = f"peer mapping unavailable ({type(e).__name__}: {str(e)[:120]})"
                    self.peerbuf = None
            # one argument list per rotating operand set (sets that together exceed L2; a single set otherwise)
            self.args, self.args_packed = [], []
            for A_t, B_t in (rot if rot is not None else [(None, None)]):
                tA, tB, tD, tb = w.tensors(A_t, B_t)
                if w.n <= 8:                             # GEMV: rows of W
                    i0, i1, a, b, d = sharding.gemv_rows(w.m, w.k, tA, tb, tD, world, rank, align=16)
                    self.args.append((capi.OP_T, capi.OP_N, i1 - i0, w.n, w.k, 1.0, a, w.k, tB, w.k, w.beta, None, 0, d, w.m, b))
                    self.block_off = i0 * es
                    if not self.args_packed:
                        # NCCL variant: the shard is written as its own packed [n, m_r] matrix and gathered rank-major
                        self.packed = torch.zeros((w.n, i1 - i0), dtype=w.D.dtype, device=dev)
                        self.gathered = torch.zeros((world, w.n, i1 - i0), dtype=w.D.dtype, device=dev)
                    dp = capi.Tensor(self.packed.data_ptr(), d.dtype, d.scale_inv, d.scale, d.amax, d.scaling)
                    self.args_packed.append(self.args[-1][:13] + (dp, i1 - i0, b))
                    self.gather_bytes = w.n * w.m * es
                else:                                    # GEMM: column blocks of B / D
                    sh = sharding.gemm_columns(w.n, w.k, w.m, w.m, tB, None, tD, world, rank)
                    self.args.append((capi.OP_T, capi.OP_N, w.m, sh.n, w.k, 1.0, tA, w.k, sh.B, w.k, w.beta, None, 0, sh.D, w.m, tb))
                    self.block_off = sh.j0 * w.m * es
                    self.cols = (sh.j0, sh.j1)
                    self.gather_bytes = w.n * w.m * es if self.needs_gather else 0
            self.amax = w.amax
        else:                                            # AdamW / casts: element chunks
            self.needs_gather = False
            i0, i1 = sharding.chunk(w.count, world, rank)
            self.range = (i0, i1)
            self.amax = w.amax

    # ---- the shard's kernel ----
    def kernel(self, i, sptr):
        w, capi = self.w, self.capi
        if w.kind == "gemm":
            if capi.gemm(*self.args[i % len(self.args)], sptr) != capi.OK:
                raise RuntimeError(capi.last_error())
        else:
            w.launch_range(sptr, *self.range)

    def kernel_bcast(self, i, sptr):
        capi = self.capi
        if capi.gemm_bcast(*self.args[i % len(self.args)], self.peerbuf.peers(self.block_off), sptr) != capi.OK:
            raise RuntimeError(capi.last_error())

    # ---- the collectives ----
    def reduce_amax(self):
        if self.amax is not None:
            self.dist.all_reduce(self.amax, op=self.dist.ReduceOp.MAX)

    def nccl_gather(self):
        if not self.needs_gather:
            return
        w = self.w
        if w.n <= 8:
            self.dist.all_gather_into_tensor(self.gathered.view(-1), self.packed.view(-1))
        else:
            flat = w.D.view(self.torch.uint8).view(-1)
            es = w.D.element_size()
            b0, b1 = self.cols[0] * w.m * es, self.cols[1] * w.m * es
            self.dist.all_gather_into_tensor(flat, flat[b0:b1])

    def step_nccl(self, i, sptr):
        """plain kernel, then NCCL all-gather of the output blocks and the amax max-all-reduce"""
        if self.w.kind == "gemm" and self.args_packed:
            if self.capi.gemm(*self.args_packed[i % len(self.args_packed)], sptr) != self.capi.OK:
                raise RuntimeError(self.capi.last_error())
        else:
            self.kernel(i, sptr)
        self.nccl_gather()
        self.reduce_amax()

    def step_fused(self, i, sptr):
        """kernel whose epilogue stores into every peer's D, then what tells every rank that all blocks have landed: the
        amax max-all-reduce where the workload has one, else the device-side flag barrier (e5b_peer_barrier: one store
        per peer and a bounded poll, no collective launched)"""
        self.kernel_bcast(i, sptr)
        if self.amax is not None:
            self.reduce_amax()
        else:
            self.peerbuf.device_barrier(sptr)


def measure_sharded(name, w, rot, tm, world, rank, dev, steps, warmup, sampler, t1_ms, min_ms=0.0):
    """kernel-only and with-collectives time of the sharded workload; T1 / (N * T_N) against the full problem on one GPU."""
    sh = Sharded(name, w, world, rank, dev, rot)
    out = {"sharding": {"c1": "column blocks of B / D", "c2": "column blocks of B / D", "c4": "column blocks of B / D (main_grad stays sharded: no collective)",
                        "c3n1": "weight rows", "c3n8": "weight rows", "c5": "parameter chunks"}.get(name, "element chunks"),
           "full_problem_one_gpu_ms": t1_ms}
    k_ms = tm.run(sh.kernel, steps, warmup, graph=True, min_ms=min_ms)
    out["kernel_only"] = {"ms_per_step": k_ms, "strong_efficiency": t1_ms / (world * k_ms)}
    has_coll = sh.needs_gather or sh.amax is not None
    best = k_ms
    # steps of a few microseconds would be timed behind the Python launch path of the collective: replay them from a
    # CUDA graph (NCCL calls capture); long steps run on the stream as before
    graph_collectives = os.environ.get("E5MA_BENCH_GRAPH_COLLECTIVES", "auto") != "0" and k_ms < 0.2
    if has_coll:
        n_ms = tm.run(sh.step_nccl, steps, warmup, graph=graph_collectives, sampler=sampler, graph_optional=True, min_ms=min_ms)
        nccl_timed_as = tm.timed_as
        out["with_collectives_nccl"] = {"ms_per_step": n_ms, "strong_efficiency": t1_ms / (world * n_ms), "timed_as": nccl_timed_as,
                                        "collectives": ("NCCL all-gather of the output (%d bytes)" % sh.gather_bytes if sh.needs_gather else "")
                                        + (" + max-all-reduce of amax" if sh.amax is not None else "")}
        best = n_ms
        if sh.peerbuf is not None:
            f_ms = tm.run(sh.step_fused, steps, warmup, graph=graph_collectives, sampler=sampler, graph_optional=True, min_ms=min_ms)
            fused_timed_as = tm.timed_as
            out["with_collectives_fused"] = {"ms_per_step": f_ms, "strong_efficiency": t1_ms / (world * f_ms), "timed_as": fused_timed_as,
                                             "collectives": "output blocks stored into every peer's D by the epilogue (e5b_gemm_bcast) + "
                                             + ("max-all-reduce of amax" if sh.amax is not None else "device-side flag barrier (e5b_peer_barrier)")}
            best = min(best, f_ms)
        elif sh.peer_note:
            out["with_collectives_fused"] = {"unavailable": sh.peer_note}
    out["ms_per_step"] = best
    return out, sh


# ---------------------------------------------------------------------------------------------------------------
ROUTE_NAMES = ["none", "gemv cp.async ring", "gemv bulk-copy ring", "tcgen05 CTA pairs 256x256", "tcgen05 CTA pairs, wide tiles",
               "tcgen05 one CTA, 256-row tiles", "tcgen05 one CTA, 128-row tiles", "CUDA cores (FP32 FMA chain)", "tcgen05 CTA pairs, mixed", "gemv row streams, FP32 FMA pipe", "gemv row streams, mma.sync",
               "tcgen05 one CTA, 256-row tiles, K split over CTA pairs", "tcgen05 one CTA, 128-row tiles, K split over CTA pairs",
               "tcgen05 one CTA, 256-row tiles, last round K-split", "tcgen05 one CTA, 128-row tiles, last round K-split"]


def gemm_rows(tm, dev, local, shrink, pk, use_graph):
    """The rows of the reference's GEMM benchmark (bench/bench_gemm.cu:33-70) at M = N = K = 4096: the four operand
    layouts of E5M2 x E5M2 -> BF16, then TN with an E4M3, BF16 and FP32 second operand and the FP32 accumulate mode.
    Each row: event-timed launches over rotating operand sets larger than L2, the kernel that ran, and the fraction
    of the peak of the unit that kernel runs on."""
    import torch
    from e5m2effma_b200 import capi, workloads
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    rows = []
    torch.cuda.synchronize()
    time.sleep(1.5)
    for name in workloads.GEMM_ROWS:
        w = None
        try:
            torch.cuda.empty_cache()
            w = workloads.make(name, dev, shrink)
            rot = rotation(w)
            samp = ClockSampler(local)
            ms = tm.run(make_step(w, rot), 20, 3, graph=use_graph, sampler=samp)
            route = capi.last_route()
            clk = samp.summary()
            tf = w.units / (ms * 1e-3) / 1e12
            if route == capi.ROUTE_SIMT:      # the reference's own yardstick: SMs x 128 FMA lanes x the SM clock of this row
                mhz = clk.get("sm_mhz") or clk.get("sm_max_mhz") or 1965
                peak, src = sms * 128 * 2 * mhz * 1e6 / 1e12, "FP32 FMA lanes at this row's SM clock"
            elif w.b_dtype in (capi.E5M2, capi.E4M3):
                peak, src = 2.0 * pk["bf16_tflops"], f"{pk['source']}: 2 x bf16_tflops burst"
            else:
                peak, src = pk["bf16_tflops"], f"{pk['source']}: bf16_tflops burst"
            rows.append({"row": workloads.GEMM_ROWS[name][0], "ms_per_step": ms, "value": tf, "unit": "TFLOP/s", "kernel": ROUTE_NAMES[route],
                         "peak": peak, "peak_source": src, "frac": tf / peak, "clocks": clk})
        except Exception as e:
            rows.append({"row": workloads.GEMM_ROWS[name][0], "error": f"{type(e).__name__}: {str(e)[:300]}"})
        finally:
            del w
    return rows


def gemv_rows(tm, dev, local, shrink, pk, use_graph):
    """The rows of the reference's GEMV benchmark (bench/bench_gemv.cu:38-47) on C3's weights (8192 x 8192 E5M2,
    row-wise scales): x in E5M2, BF16 and FP32, batch 1, 2, 4, 8.  GB/s of algorithmic bytes (W once, x, scales, y)."""
    import torch
    from e5m2effma_b200 import capi, workloads
    rows = []
    torch.cuda.synchronize()
    time.sleep(1.5)
    for name in workloads.GEMV_ROWS:
        w = None
        try:
            torch.cuda.empty_cache()
            w = workloads.make(name, dev, shrink)
            samp = ClockSampler(local)
            ms = tm.run(make_step(w, rotation(w)), 20, 3, graph=use_graph, sampler=samp)
            gbs = w.units / (ms * 1e-3) / 1e9
            rows.append({"row": workloads.GEMV_ROWS[name][0], "ms_per_step": ms, "value": gbs, "unit": "GB/s", "kernel": ROUTE_NAMES[capi.last_route()],
                         "peak": pk["hbm_gbs"], "peak_source": f"{pk['source']}: hbm_gbs (copy)", "frac": gbs / pk["hbm_gbs"], "clocks": samp.summary()})
        except Exception as e:
            rows.append({"row": workloads.GEMV_ROWS[name][0], "error": f"{type(e).__name__}: {str(e)[:300]}"})
        finally:
            del w
    return rows


def run_reference(args, metric, unit, config):
    """The reference's CPU algorithm (oracle port) on the same seeded inputs, all host threads; rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    import torch
    import oracle as orc
    from e5m2effma_b200 import workloads

    def cpu_quantizer(x32, dtype, scale=None):
        codes = orc.encode(dtype, x32.detach().float().cpu().contiguous().numpy().reshape(-1), 1.0 if scale is None else float(scale))
        return torch.from_numpy(codes.reshape(tuple(x32.shape))).to(x32.device)

    workloads.QUANTIZER = cpu_quantizer              # the library is not loaded in this arm
    name = args.workload
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if torch.cuda.is_available() else torch.device("cpu")
    gen_note = ("inputs: the GPU arm's seeds and torch CUDA generator, quantised by the oracle's encoder (bit-identical to e5ma_cast)"
                if dev.type == "cuda" else "inputs: the GPU arm's seeds and distributions drawn with torch's CPU generator (no GPU visible)")
    shrink = args.shrink
    if name == "c2":
        w = workloads.make("c2_bf16", dev, shrink)
        hg = HostGemm(w, d_dtype=orc.BF16)
        _, slab_amax = hg.timed_slab(orc, (0, 4))    # untimed first pass over a few columns supplies prev_amax
        w.d_dtype = orc.E5M2
        hg = HostGemm(w, d_dtype=orc.E5M2, d_scale=57344.0 / max(float(slab_amax), 1e-30))
        kw = {"hg": hg}
    elif name == "c5":
        w = workloads.AdamWorkload("c5", (1 << 26) // shrink, dev, seed=5000)
        w.count = (1 << 30) // shrink
        kw = {}
    elif name.startswith("cast"):
        src_dst = {"cast_f32_e5m2": (orc.FP32, orc.E5M2, 6000), "cast_bf16_e4m3": (orc.BF16, orc.E4M3, 6100), "cast_e4m3_bf16": (orc.E4M3, orc.BF16, 6200)}[name]
        w = workloads.CastWorkload(name, (1 << 27) // shrink, src_dst[0], src_dst[1], dev, seed=src_dst[2])
        kw = {}
    else:
        w = workloads.make(name, dev, shrink)
        kw = {"hg": HostGemm(w)}
    vals, secs, sample = [], [], ""
    for i in range(args.warmup + args.steps):
        v, u, sample, t1 = cpu_sample(w, orc, 4.0, **kw) if w.kind == "gemm" else cpu_sample(w, orc, 4.0)
        if i >= args.warmup:
            vals.append(v)
            secs.append(t1)
    val = sum(vals) / len(vals)
    ms = sum(secs) * 1e3 / len(secs)
    line = {"impl": "reference", "metric": metric, "value": val, "unit": unit, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong" if args.gpus > 1 else "weak",
            "vs_baseline": None, "dtype": "f32 chain (CPU)", "data": "synthetic", "config": config,
            "cpu_baseline": {"value": val, "unit": unit, "cores": orc.threads(), "kind": "port", "sample": sample + "; " + gen_note},
            "e2e": {"value": val, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "reference GPU kernels refuse sm_89+ (src/e5m2effma.cuh:22-26); its host emulation is inline in its tests, "
                    "so the CPU oracle port of that emulation is timed"}
    print(json.dumps(line), flush=True)


def e2e_single(w, tm, steps, scale_div):
    """N = 1 end to end: every step uploads all inputs from pinned host memory, calls the C interface and reads the
    result back; two buffer sets and three streams overlap the copies of neighbouring steps with the kernel."""
    import torch
    stream = tm.stream
    ins, outs = w.io_tensors()
    outs = [t for t in outs if t is not None]
    host_in = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True).copy_(t) for t in ins]
    host_out = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True) for t in outs]
    h2d = sum(t.numel() * t.element_size() for t in ins)
    d2h = sum(t.numel() * t.element_size() for t in outs)
    sets = []
    for b in range(2):
        if w.kind == "gemm":
            dA, dB, dD = (w.A, w.B, w.D) if b == 0 else (w.A.clone(), w.B.clone(), w.D.clone())
            swap = {id(w.A): dA, id(w.B): dB, id(w.D): dD}
            sets.append({"ins": [swap.get(id(t), t) for t in ins], "outs": [swap.get(id(t), t) for t in outs],
                         "launch": (lambda st, a=dA, bb=dB, d=dD: w.launch(st, a, bb, d))})
        else:
            sets.append({"ins": ins, "outs": outs, "launch": (lambda st: w.launch(st))})
    s_in, s_run, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_run = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]
    for e in ev_run + ev_out:
        e.record(stream)

    def step(i):
        b = i & 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_run[b])
            for d, h in zip(sets[b]["ins"], host_in):
                d.copy_(h, non_blocking=True)
            ev_in[b].record(s_in)
        with torch.cuda.stream(s_run):
            s_run.wait_event(ev_in[b])
            s_run.wait_event(ev_out[b])
            sets[b]["launch"](s_run.cuda_stream)
            ev_run[b].record(s_run)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_run[b])
            for h, d in zip(host_out, sets[b]["outs"]):
                h.copy_(d, non_blocking=True)
            ev_out[b].record(s_out)

    def join():
        for st in (s_in, s_run, s_out):
            stream.wait_stream(st)

    ksteps = max(4, min(steps, 10))
    for st in (s_in, s_run, s_out):
        st.wait_stream(stream)
    for i in range(2):
        step(i)
    join()
    tm.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for st in (s_in, s_run, s_out):
        st.wait_stream(stream)
    for i in range(ksteps):
        step(i)
    join()
    e1.record(stream)
    tm.barrier()
    ems = e0.elapsed_time(e1)
    return {"value": w.units / (ems / ksteps * 1e-3) / scale_div, "unit": None, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "ms_per_step": ems / ksteps, "steps": ksteps, "pipeline": "2 buffer sets, upload / kernel / read-back on separate streams"}


def e2e_sharded(sh, tm, steps, scale_div):
    """N > 1 end to end for a column-sharded GEMM: every step, each rank uploads ITS 1/N of A, its block of B and the
    small vectors from pinned host memory, A is completed over NVLink (NCCL all-gather: "A broadcast" without N
    copies over PCIe), the rank computes its block of D (stored into every peer's D by the epilogue when peer
    mappings exist, else NCCL all-gather), amax is max-reduced, and the rank reads its block of D and the amax back."""
    import torch
    import torch.distributed as dist
    w, world, rank = sh.w, sh.world, sh.rank
    stream = tm.stream
    rows = w.m // world
    a_part = w.A[rank * rows:(rank + 1) * rows]
    b_part = w.B[sh.cols[0]:sh.cols[1]]
    d_part = w.D[sh.cols[0]:sh.cols[1]]
    small = [t for t in (w.sa, w.sb, w.bias) if t is not None]
    ins = [a_part, b_part] + small
    outs = [d_part] + ([w.amax] if w.amax is not None else [])
    host_in = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True).copy_(t) for t in ins]
    host_out = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True) for t in outs]
    h2d = sum(t.numel() * t.element_size() for t in ins)
    d2h = sum(t.numel() * t.element_size() for t in outs)
    a_flat = w.A.view(-1)

    def step(i):
        for d, h in zip(ins, host_in):
            d.copy_(h, non_blocking=True)
        dist.all_gather_into_tensor(a_flat, a_part.reshape(-1))
        if sh.peerbuf is not None:
            sh.step_fused(i, stream.cuda_stream)
        else:
            sh.step_nccl(i, stream.cuda_stream)
        for h, d in zip(host_out, outs):
            h.copy_(d, non_blocking=True)

    ksteps = max(4, min(steps, 10))
    for i in range(2):
        step(i)
    tm.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(ksteps):
        step(i)
    e1.record(stream)
    tm.barrier()
    ems = tm.max_over_ranks(e0.elapsed_time(e1))
    return {"value": w.units / (ems / ksteps * 1e-3) / scale_div, "unit": None, "h2d_bytes_per_step": h2d * world,
            "d2h_bytes_per_step": d2h * world, "h2d_bytes_per_step_per_rank": h2d, "d2h_bytes_per_step_per_rank": d2h,
            "ms_per_step": ems / ksteps, "steps": ksteps,
            "pipeline": "per rank: upload 1/N of A + own block of B, NCCL all-gather of A over NVLink, sharded GEMM with the "
                        + ("epilogue storing into every peer's D" if sh.peerbuf is not None else "NCCL all-gather of D")
                        + ", amax max-all-reduce, read-back of the rank's block of D; one stream, steps not overlapped"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c2")
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--shrink", type=int, default=1, help="divide the problem sizes (profiler captures)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="headline workload only (no workloads section, no sustained loop)")
    ap.add_argument("--no-graph", action="store_true", help="launch the timed steps one by one instead of as one CUDA graph")
    ap.add_argument("--sustain-s", type=float, default=2.0, help="length of the sustained-regime loop of the headline workload")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl != "reference" else args.warmup
    name = args.workload
    is_flops = name in GEMM_LIKE
    metric = METRIC.get(name, name)
    unit = "TFLOP/s" if is_flops else "GB/s"
    world = int(os.environ.get("WORLD_SIZE", "1"))
    config = {"workload": DESC.get(name, name),
              "problem": ("the stated problem, sharded over the ranks (strong scaling): " if world > 1 else "") +
                         "column blocks of B / D for GEMMs, weight rows for the GEMV, element chunks for AdamW / casts",
              "l2": "inputs larger than L2 (126 MB)" if name not in ("c1", "c3n1", "c3n8") else "rotating input sets larger than L2"}
    if world > 1:      # the same text in both arms: the figure itself is the top-level key "weak_scaling" of the GPU arm's line
        config["weak"] = "weak-scaling figure (every rank the full problem, amax reduced every step): top-level key weak_scaling"
    if args.impl == "reference":
        run_reference(args, metric, unit, config)
        return

    import torch
    import torch.distributed as dist
    from e5m2effma_b200 import capi

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a GPU (the library has no CPU path)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    pk = peaks()
    tm = Timing(dev, world)
    sampler = ClockSampler(local)
    scale_div = 1e12 if is_flops else 1e9
    use_graph = not args.no_graph

    err_cols = None
    if world == 1 and not args.no_cpu and name in GEMM_LIKE:
        n_full = {"c1": 4096, "c2": 4096, "c4": 4096}[name] // args.shrink
        err_cols = [(0, 4), (n_full // 2 - 2, n_full // 2 + 2)]
    w, first_pass_cols = build_workload(name, dev, args.shrink, world, keep_first_pass=err_cols if name == "c2" else None)
    rot = rotation(w, world)
    step_full = make_step(w, rot)

    # ---- the full problem on one GPU (the headline at N = 1; T_1 of the strong-scaling figures at N > 1) ----
    t1_ms = tm.run(step_full, args.steps, args.warmup, graph=use_graph, sampler=sampler if world == 1 else None)
    clocks = sampler.summary()
    fault = capi.gemm_fault()
    line_extra = {}

    if world == 1:
        ms_per_step = t1_ms
        value = w.units / (ms_per_step * 1e-3) / scale_div
        roof = roofline(name, w, ms_per_step, pk)
        scaling = "weak"
        launches = args.steps * w.launches_per_pass
        timed_as = "cuda_graph" if use_graph else "stream"
    else:
        # weak figure first (every rank the full problem, amax max-reduced after every step), then the sharded problem
        def weak_step(i, sptr):
            step_full(i, sptr)
            if getattr(w, "amax", None) is not None:
                dist.all_reduce(w.amax, op=dist.ReduceOp.MAX)
        weak_ms = tm.run(weak_step, args.steps, args.warmup, graph=False)
        line_extra["weak_scaling"] = {"ms_per_step": weak_ms, "value": w.units * world / (weak_ms * 1e-3) / scale_div, "unit": unit,
                                      "what": "every rank runs the full problem; one max-all-reduce of amax per step"}
        sharded, sh = measure_sharded(name, w, rot, tm, world, rank, dev, args.steps, args.warmup, sampler, t1_ms)
        ms_per_step = sharded["ms_per_step"]
        value = w.units / (ms_per_step * 1e-3) / scale_div
        roof = roofline(name, w, sharded["kernel_only"]["ms_per_step"], pk, units=w.units / world)
        roof["note"] = "per GPU: the shard's kernel alone (algorithmic work / N) against one GPU's peak"
        line_extra["strong_scaling"] = sharded
        scaling = "strong"
        launches = args.steps * w.launches_per_pass
        timed_as = "stream (collectives inside every step)"
        clocks = sampler.summary()

    # ---- end to end ----
    e2e = None
    if not args.no_e2e:
        if world == 1:
            bg = ClockSampler(local)
            bg.start()
            e2e = e2e_single(w, tm, args.steps, scale_div)
            bg.stop_flag = True
            bg.join()
        elif w.kind == "gemm" and w.n > 8:
            e2e = e2e_sharded(sh, tm, args.steps, scale_div)
        if e2e is not None:
            e2e["unit"] = unit

    # ---- the other configurations of the metric ----
    others = None
    if not args.no_extras and name == "c2":
        others = {}
        for other in EXTRAS:
            del_w = None
            try:
                torch.cuda.empty_cache()
                ow, _ = build_workload(other, dev, args.shrink, world)
                del_w = ow
                orot = rotation(ow, world)
                ostep = make_step(ow, orot)
                osamp = ClockSampler(local)
                steps_o = min(args.steps, 20)
                torch.cuda.synchronize()
                time.sleep(1.5)     # the burst figure of each workload starts from an idle, cooled-off GPU like the headline's
                o_t1 = tm.run(ostep, steps_o, 3, graph=use_graph, sampler=osamp if world == 1 else None)
                odiv = 1e12 if other in GEMM_LIKE else 1e9
                ounit = "TFLOP/s" if other in GEMM_LIKE else "GB/s"
                if world == 1:
                    entry = {"workload": DESC.get(other, other), "ms_per_step": o_t1, "value": ow.units / (o_t1 * 1e-3) / odiv, "unit": ounit,
                             "roofline": roofline(other, ow, o_t1, pk), "clocks": osamp.summary(), "steps": steps_o}
                    if other in ("c1", "c4"):
                        s_ms, s_clk, s_l = tm.sustained(ostep, o_t1, ClockSampler(local), 1.0)
                        entry["roofline"]["sustained"] = sustained_entry(other, ow, s_ms, s_clk, s_l, pk)
                        if not args.no_cpu and rank == 0:
                            import oracle as orc
                            entry["observed_error"] = error_report(ow, orc, [(0, 4), (ow.n // 2 - 2, ow.n // 2 + 2)])
                else:
                    shd, _ = measure_sharded(other, ow, orot, tm, world, rank, dev, steps_o, 3, osamp, o_t1, min_ms=3.0)
                    entry = {"workload": DESC.get(other, other), "ms_per_step": shd["ms_per_step"],
                             "value": ow.units / (shd["ms_per_step"] * 1e-3) / odiv, "unit": ounit, "strong_scaling": shd,
                             "roofline": roofline(other, ow, shd["kernel_only"]["ms_per_step"], pk, units=ow.units / world), "steps": steps_o}
                others[other] = entry
            except Exception as e:      # one workload failing must not lose the headline
                others[other] = {"error": f"{type(e).__name__}: {str(e)[:300]}"}
            finally:
                del del_w
        fault = fault or capi.gemm_fault()

    # ---- the layout and pairing rows of the reference's GEMM benchmark (N = 1) ----
    rows = None
    if world == 1 and not args.no_extras and name == "c2":
        rows = gemm_rows(tm, dev, local, args.shrink, pk, use_graph) + gemv_rows(tm, dev, local, args.shrink, pk, use_graph)
        fault = fault or capi.gemm_fault()

    # ---- sustained regime of the headline (N = 1) ----
    if world == 1 and not args.no_extras and args.sustain_s > 0:
        s_ms, s_clk, s_launches = tm.sustained(step_full, t1_ms, ClockSampler(local), args.sustain_s)
        roof["sustained"] = sustained_entry(name, w, s_ms, s_clk, s_launches, pk)

    def finish():
        """Leave without tearing NCCL down (destroying the process group after graph captures has hung at exit)."""
        sys.stdout.flush()
        sys.stderr.flush()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
            os._exit(0)

    if rank != 0:
        finish()
        return

    cpu = None
    if world == 1 and not args.no_cpu:
        import oracle as orc
        if w.kind == "gemm":
            hg = HostGemm(w)
            v, u, sample, _ = cpu_gemm(w, orc, 12.0, hg=hg)
        else:
            v, u, sample, _ = cpu_sample(w, orc, 12.0)
        cpu = {"value": v, "unit": u, "cores": orc.threads(), "kind": "port", "sample": sample}
        if err_cols is not None:
            cpu["observed_error"] = error_report(w, orc, err_cols, first_pass=first_pass_cols)
            if name == "c2" and "output" in cpu["observed_error"]:
                cpu["observed_error"]["output"]["pass"] = "first pass of the same operands with BF16 output (the one that supplies prev_amax)"

    line = {"metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
            "dtype": DTYPE.get(name, "f32"), "data": "synthetic", "config": config, "clocks": clocks, "e2e": e2e,
            "gpu_launches": launches, "timed_as": timed_as, "roofline": roof, "cpu_baseline": cpu, "tolerance": TOLERANCE,
            "gemm_fault": fault}
    line.update(line_extra)
    if others is not None:
        line["workloads"] = others
    if rows is not None:
        line["gemm_rows"] = rows
    print(json.dumps(line), flush=True)
    finish()


if __name__ == "__main__":
    main()
