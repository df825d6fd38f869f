#!/usr/bin/env python
"""Benchmark of the hot path through the C interface.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One "step" is one pass of the chosen workload (default: c2, the HYBRID dgrad GEMM
8192 x 4096 x 14336, E5M2 row-wise x E4M3 + BF16 bias -> E5M2 + amax) over synthetic, seeded
inputs.  One JSON line goes to stdout:

  value      whole-job throughput with the inputs resident in HBM (TFLOP/s for GEMMs, GB/s for
             the bandwidth-bound workloads), timed with CUDA events on the launching stream over
             exactly K steps, max over ranks
  e2e        the same metric with the step's inputs starting in pinned host memory: host-to-device
             copies, the call through the C interface and the device-to-host read of the result
             are all inside the timed region
  roofline   algorithmic FLOPs (or bytes) per launch / average launch time, against the measured
             peak of MEASURED_PEAKS.json (FP8: twice the measured BF16 figure)
  cpu_baseline  the CPU oracle (a restatement of the reference's host emulation) on a bounded sample
             of the same workload, all host threads (rank 0, N = 1 only)

Multi-GPU: launched under torchrun, one rank per GPU.  The GEMM is sharded by column blocks of B
with A replicated (weak scaling: every rank keeps the full per-GPU problem), the only data-path
collective is the max-all-reduce of the scalar amax; AdamW / casts shard by parameter chunks,
the GEMV by weight rows.

--impl reference times the reference's own CPU algorithm (the oracle port: the reference's GPU
kernels refuse this architecture and its host emulation does not build stand-alone) on the same
configuration and prints the same line with "impl": "reference".
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

# DRAM traffic per launch (dram__bytes_read.sum + dram__bytes_write.sum) from the ncu captures
# summarised under profiles/; None where no capture has been taken.
NCU_TRAFFIC_BYTES = {
    "c2": 434.7e6,     # profiles/gemm_tc_pair_kernel__c2_hybrid_dgrad.md (full size)
    "c1": 34.5e6,      # profiles/gemm_tc_pair_kernel__c1_4096cube.md (full size, operands fit L2)
    "c4": 1943.0e6,    # profiles/gemm_tc_kernel__c4_wgrad_mixed.md (full size)
    "c3n1": 68.1e6,    # profiles/gemv_async_kernel__c3_batch1.md (full size)
    "c3n8": 67.8e6,    # profiles/gemv_async_kernel__c3_batch8.md
    "c5": 15.65e9,     # profiles/adam_kernel__c5_shrunk8.md: 1.956 GB at 2^27 elements, scaled x8 (traffic is linear in the count)
    "cast_e4m3_bf16": 2.994e9,   # profiles/cast_kernel__e4m3_to_bf16_shrunk4.md: 748.4 MB at 2^28 elements, scaled x4
}

GEMM_LIKE = ("c1", "c2", "c4")


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "bf16_tflops_sustained": p.get("bf16_tflops_sustained"),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs (read-only)."""

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
        `event` has completed.  Used for the device-resident region: a sampling thread beside the thread that
        launches delays launches now and then, and with a collective in every step all ranks pay for each
        such delay (measured at N = 8: 0.59-0.70 ms per step with the thread, 0.36 ms without)."""
        self.sample()
        while not event.query():
            self.sample()
            time.sleep(0.0005)

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


def cpu_sample(name, target_s=12.0):
    """The CPU oracle on a bounded sample of workload `name`; returns (value, unit, description, seconds)."""
    import numpy as np
    import oracle as orc
    rng = np.random.default_rng(1234)
    if name in GEMM_LIKE or name.startswith("c3"):
        shapes = {"c1": (4096, 4096, 4096), "c2": (8192, 4096, 14336), "c4": (4096, 4096, 65536),
                  "c3n1": (8192, 1, 8192), "c3n8": (8192, 8, 8192)}
        m, n, k = shapes[name]
        bt = orc.BF16 if name in ("c4", "c3n1", "c3n8") else (orc.E4M3 if name == "c2" else orc.E5M2)
        A = rng.integers(0, 120, m * k).astype(np.uint8)
        # bounded sample: full rows and full k, as many output columns as the MAC budget allows
        budget = target_s * 1.2e11
        cols = n if n <= 8 else int(min(n, max(8, budget // (m * k)))) // 4 * 4

        def run(ncols):
            B = rng.integers(0, 120, ncols * k).astype(np.uint8) if bt != orc.BF16 else \
                orc.encode(orc.BF16, rng.standard_normal(ncols * k).astype(np.float32))
            D = np.zeros(m * ncols, np.uint16)
            t = time.perf_counter()
            orc.gemm(1, 0, m, ncols, k, 1.0, A, orc.E5M2, k, B, bt, k, 0.0, None, orc.FP32, m, D, orc.BF16, m,
                     a_sinv=0.125, b_sinv=0.125)
            return time.perf_counter() - t

        t1 = run(cols)
        if name.startswith("c3"):
            return (m * k + 2.0 * k * cols) / t1 / 1e9, "GB/s", f"all {m} rows, {cols} of {n} columns, full k = {k}: {t1:.2f} s", t1
        return 2.0 * m * cols * k / t1 / 1e12, "TFLOP/s", f"all {m} rows, {cols} of {n} output columns, full k = {k}: {t1:.2f} s", t1
    if name == "c5":
        cnt = 1 << 26
        p = orc.encode(orc.BF16, (rng.standard_normal(cnt) * 0.02).astype(np.float32))
        g = orc.encode(orc.BF16, (rng.standard_normal(cnt) * 1e-3).astype(np.float32))
        mm, vv, q = np.zeros(cnt, np.uint16), np.zeros(cnt, np.uint16), np.zeros(cnt, np.uint8)
        cfg = dict(lr=3e-4, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.1, step=1, adamw=1, bias_correction=1, grad_scale=1.0)
        t = time.perf_counter()
        orc.adam(cfg, p, orc.BF16, g, orc.BF16, mm, vv, orc.BF16, q, orc.E4M3, 2048.0, 0.0)
        t1 = time.perf_counter() - t
        return cnt * 15.0 / t1 / 1e9, "GB/s", f"2^26 of 2^30 parameters: {t1:.2f} s", t1
    es = {"cast_f32_e5m2": (orc.FP32, orc.E5M2, 5), "cast_bf16_e4m3": (orc.BF16, orc.E4M3, 3), "cast_e4m3_bf16": (orc.E4M3, orc.BF16, 3)}[name]
    cnt = 1 << 27
    src = rng.standard_normal(cnt).astype(np.float32) if es[0] == orc.FP32 else \
        (rng.integers(0, 120, cnt).astype(np.uint8) if es[0] == orc.E4M3 else rng.integers(0, 2 ** 15, cnt).astype(np.uint16))
    t = time.perf_counter()
    orc.cast(src, es[0], es[1], 0.5, 16.0, amax=0.0)
    t1 = time.perf_counter() - t
    return cnt * es[2] / t1 / 1e9, "GB/s", f"2^27 elements: {t1:.2f} s", t1


def parity_sample(w, orc):
    """Part of the cpu_baseline leg: the oracle re-computes a few output columns (all rows, full k) of the
    result the GPU just produced and reports the largest error in units of the stated bound
    (1 ulp of the output format is allowed on top: a ratio <= 1 is inside the bound without it)."""
    import numpy as np
    import torch
    st = {0: np.uint8, 4: np.uint8, 1: np.uint16, 2: np.uint16, 3: np.float32}

    def host(t):
        return t.detach().cpu().contiguous().view(torch.uint8).numpy()

    w.launch(torch.cuda.current_stream().cuda_stream)      # a fresh result from the original operands
    torch.cuda.synchronize()
    A, B = host(w.A).view(st[w.a_dtype]).reshape(-1), host(w.B).view(st[w.b_dtype]).reshape(-1)
    D = host(w.D).view(st[w.d_dtype]).reshape(w.n, w.m)
    if w.beta != 0.0:
        return {"skipped": "accumulating workload: the timed steps have already changed D"}
    qs = float(w.d_scale.item()) if w.d_scale is not None else 1.0
    cols = [(0, min(4, w.n)), (max(0, w.n // 2 - 2), min(w.n, w.n // 2 + 2))] if w.n > 8 else [(0, w.n)]
    worst = 0.0
    for j0, j1 in cols:
        ref, mag, fix = orc.gemm_wide(1, 0, w.m, w.n, w.k, 1.0, A, w.a_dtype, w.k, B, w.b_dtype, w.k, 0.0, None, w.d_dtype, w.m,
                                      bias=None if w.bias is None else host(w.bias).view(np.uint16), bias_dtype=orc.BF16,
                                      a_sinv=None if w.sa is None else w.sa.cpu().numpy(), a_outer=w.a_outer,
                                      b_sinv=None if w.sb is None else w.sb.cpu().numpy(), b_outer=w.b_outer, cols=(j0, j1))
        got = orc.decode(w.d_dtype, D[j0:j1].copy(), 1.0).astype(np.float64) / qs
        # one ulp of the output format around the reference, then the accumulation-order bound
        ulp = {0: 2.0 ** -3, 4: 2.0 ** -2, 1: 2.0 ** -7, 2: 2.0 ** -10, 3: 2.0 ** -23}[w.d_dtype] * np.maximum(np.abs(ref), 1e-30)
        bound = w.k * 2.0 ** -23 * mag + 2.0 ** -21 * (np.abs(ref) + fix + mag)
        excess = np.maximum(np.abs(got - ref) - ulp, 0.0) / np.maximum(bound, 1e-300)
        worst = max(worst, float(excess.max()))
    return {"columns": sum(b - a for a, b in cols), "rows": w.m, "bound": "k * 2^-23 * sum|a*b|*|s| beyond 1 ulp of the output format",
            "max_error_over_bound": worst, "ok": worst <= 1.0}


def run_reference(args, metric, unit, config):
    """The reference's CPU algorithm (oracle port) on this configuration, all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle as orc
    vals, secs = [], []
    for i in range(args.warmup + args.steps):
        v, u, sample, t1 = cpu_sample(args.workload, target_s=4.0)
        if i >= args.warmup:
            vals.append(v)
            secs.append(t1)
    val = sum(vals) / len(vals)
    ms = sum(secs) * 1e3 / len(secs)            # the oracle call alone; generating the sample's inputs is untimed
    line = {"impl": "reference", "metric": metric, "value": val, "unit": unit, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32 chain (CPU)", "data": "synthetic", "config": config,
            "cpu_baseline": {"value": val, "unit": unit, "cores": orc.threads(), "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "reference GPU kernels refuse sm_89+ (src/e5m2effma.cuh:22-26); its host emulation is inline in its tests, "
                    "so the CPU oracle port of that emulation is timed"}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--settle-s", type=float, default=0.0,
                    help="N > 1 with a collective in the step: seconds of untimed steps after the warm-up, until the "
                         "power-capped clocks have settled")
    ap.add_argument("--amax-reduce", default="inline", choices=["inline", "fused", "overlap", "off"],
                    help="N > 1: how the per-step amax is max-reduced over the ranks (see the comment in main())")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c2")
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--shrink", type=int, default=1, help="divide the problem sizes (profiler captures)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch the timed steps one by one instead of as one CUDA graph")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl != "reference" else args.warmup
    name = args.workload
    is_flops = name in GEMM_LIKE
    metric = {"c1": "fp8_gemm_4096_e5m2_bf16", "c2": "fp8_hybrid_dgrad_gemm", "c4": "wgrad_e5m2_bf16_fp32_accumulate",
              "c3n1": "gemv_8192_e5m2_bf16_batch1", "c3n8": "gemv_8192_e5m2_bf16_batch8", "c5": "fused_adamw_bf16_e4m3_copy"}.get(name, name)
    unit = "TFLOP/s" if is_flops else "GB/s"
    desc = {"c1": "GEMM M=N=K=4096 E5M2 x E5M2 (TN, scale_inv 0.125) -> BF16",
            "c2": "HYBRID dgrad GEMM M=8192 N=4096 K=14336, E5M2 row-wise x E4M3 per-tensor + BF16 bias -> E5M2 + amax",
            "c3n1": "decode GEMV W 8192x8192 E5M2 row-wise, x BF16 batch 1 -> BF16",
            "c3n8": "decode GEMV W 8192x8192 E5M2 row-wise, x BF16 batch 8 -> BF16",
            "c4": "wgrad GEMM M=N=4096 K=65536 E5M2 x BF16, beta=1 into FP32 main_grad",
            "c5": "fused AdamW over 2^30 BF16 parameters, BF16 m/v, E4M3 copy + amax"}.get(name, name)
    config = {"workload": desc, "per_gpu_problem": "full (weak scaling: column blocks / rows / chunks per rank)",
              "l2": "inputs larger than L2 (126 MB)" if name not in ("c1", "c3n1", "c3n8") else "rotating input sets larger than L2"}
    if args.impl == "reference":
        run_reference(args, metric, unit, config)
        return

    import torch
    import torch.distributed as dist
    from e5m2effma_b200 import capi, workloads

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a GPU (the library has no CPU path)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    # ---- inputs -----------------------------------------------------------------------------------
    if name == "c2":
        first = workloads.make("c2_bf16", dev, args.shrink)      # BF16 pass that supplies prev_amax
        first.launch(torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        prev_amax = float(first.amax.item())
        if world > 1:
            t = first.amax.clone()
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            prev_amax = float(t.item())
        w = first
        w.d_dtype = capi.E5M2
        w.D = torch.zeros((w.n, w.m), dtype=torch.uint8, device=dev)
        workloads.finish_c2(w, prev_amax)
    else:
        w = workloads.make(name, dev, args.shrink)
    stream = torch.cuda.current_stream()
    sptr = stream.cuda_stream

    # workloads whose operands fit in L2 rotate over input sets that together exceed it
    rot = None
    if w.kind == "gemm" and (w.A.numel() * w.A.element_size() + w.B.numel() * w.B.element_size()) < 200e6:
        sets = int(260e6 // (w.A.numel() * w.A.element_size() + w.B.numel() * w.B.element_size())) + 1
        rot = [(w.A.clone(), w.B.clone()) for _ in range(sets)]

    def one_pass(i):
        if rot is not None:
            a, b = rot[i % len(rot)]
            w.launch(sptr, a, b)
        else:
            w.launch(sptr)

    # N > 1: every step's amax is max-reduced over the ranks, inside the timed region.  Modes (--amax-reduce):
    #   inline   (default) one all-reduce of one float after every step;
    #   fused    step i writes its amax into slot i of a vector and ONE all-reduce over the vector follows the last
    #            step -- what delayed-scaling recipes do once per iteration for all their tensors; the per-step
    #            figure is then also timed after the main region and reported beside the value;
    #   overlap  the reduction of step i runs beside step i + 1 (two slots alternate); no faster than inline at
    #            N = 2: the persistent GEMM sizes its grid to every SM, and a reduction kernel that holds an SM
    #            when the next GEMM starts delays one of its CTA pairs;
    #   off      no reduction (experiments).
    # With a reduction in the step the K steps are launched on the stream, not replayed from a CUDA graph (a step of
    # a third of a millisecond hides the launch path; at N = 8: 0.36 ms per step, 0.35 ms without any reduction).
    amax_t = getattr(w, "amax", None)
    mode = args.amax_reduce
    reduce_amax = world > 1 and amax_t is not None and mode != "off"
    amax_slots = [amax_t, amax_t.clone()] if reduce_amax else None
    amax_vec = torch.zeros(max(args.steps, args.warmup, 1), dtype=torch.float32, device=dev) if reduce_amax else None
    pending = []

    def step(i):
        if reduce_amax and mode == "overlap":
            if len(pending) == 2:
                pending.pop(0).wait()
            w.amax = amax_slots[i % 2]
        elif reduce_amax and mode == "fused":
            j = i % amax_vec.numel()
            w.amax = amax_vec[j:j + 1]
        one_pass(i)
        if reduce_amax and mode == "overlap":
            pending.append(dist.all_reduce(w.amax, op=dist.ReduceOp.MAX, async_op=True))
        elif reduce_amax and mode == "inline":
            dist.all_reduce(w.amax, op=dist.ReduceOp.MAX)

    def drain():
        while pending:
            pending.pop(0).wait()
        if reduce_amax and mode == "fused":
            dist.all_reduce(amax_vec, op=dist.ReduceOp.MAX)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing -------------------------------------------------------------------
    # The K timed steps are captured once into a CUDA graph and replayed, so that microsecond-scale
    # kernels (the 4096^3 GEMM, the GEMV) are not timed behind the Python / ctypes launch path.
    # NVML is initialised here, not between the warm-up and the timed steps: the GPUs must not idle there (with a
    # collective in every step, N GPUs that ramp their clocks up again each at its own pace cost every step)
    sampler = ClockSampler(local)
    w0, w1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    w0.record(stream)
    for i in range(args.warmup):
        step(i)
    drain()
    w1.record(stream)
    barrier()
    settle_steps = 0
    if reduce_amax and args.settle_s > 0:
        # Optional (off by default): untimed steps until the power-capped clocks have settled, to measure the
        # sustained regime (C2 at N = 2: 0.44 ms per step at 1.41 GHz against 0.35 ms in the first milliseconds).
        # Every rank derives the same count from the all-reduced warm-up time.
        t = torch.tensor([w0.elapsed_time(w1) / max(args.warmup, 1)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        settle_steps = int(min(8000, args.settle_s * 1e3 / max(float(t.item()), 1e-3)))
        for i in range(settle_steps):
            step(i)
        drain()
        barrier()
    graph = None
    if not args.no_graph and not reduce_amax:
        cs = torch.cuda.Stream()
        cs.wait_stream(stream)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(cs):
            sptr_saved, sptr = sptr, cs.cuda_stream
            with torch.cuda.graph(graph, stream=cs):
                for i in range(args.steps):
                    step(i)
                drain()
            sptr = sptr_saved
        graph.replay()          # one untimed replay (also warms the instantiated graph)
        barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    if graph is not None:
        graph.replay()
    else:
        for i in range(args.steps):
            step(i)
        drain()
    e1.record(stream)
    sampler.poll_until(e1)      # the GPU is still working through the timed steps: clocks under load
    barrier()
    ms = e0.elapsed_time(e1)
    inline_aux = None
    if reduce_amax:
        torch.maximum(amax_slots[0], amax_slots[1], out=amax_slots[0])
        torch.maximum(amax_t, amax_vec.max().reshape(1), out=amax_t)
        w.amax = amax_t
        if mode == "fused":      # the same K steps with one all-reduce per step, for the record
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            for i in range(3):
                one_pass(i)
                dist.all_reduce(amax_t, op=dist.ReduceOp.MAX)
            barrier()
            a0.record(stream)
            for i in range(args.steps):
                one_pass(i)
                dist.all_reduce(amax_t, op=dist.ReduceOp.MAX)
            a1.record(stream)
            barrier()
            t = torch.tensor([a0.elapsed_time(a1)], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            inline_aux = float(t.item()) / args.steps
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / args.steps
    scale_div = 1e12 if is_flops else 1e9
    value = w.units * world / (ms_per_step * 1e-3) / scale_div
    fault = capi.gemm_fault()

    # ---- end to end: pinned host inputs -> device -> call -> result back --------------------------
    e2e = None
    if not args.no_e2e:
        sampler.start()          # the end-to-end region is host-paced anyway: a sampling thread runs beside it
        ins, outs = w.io_tensors()
        outs = [t for t in outs if t is not None]
        host_in = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True).copy_(t) for t in ins]
        host_out = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True) for t in outs]
        h2d = sum(t.numel() * t.element_size() for t in ins)
        d2h = sum(t.numel() * t.element_size() for t in outs)

        # Two sets of device buffers and three streams: the upload of step i+1 and the read-back of step i-1
        # overlap the kernel of step i.  Every step still moves all of its inputs and its result.
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

        def e2e_step(i):
            b = i & 1
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_run[b])          # the kernel that last read this buffer set is done
                for d, h in zip(sets[b]["ins"], host_in):
                    d.copy_(h, non_blocking=True)
                ev_in[b].record(s_in)
            with torch.cuda.stream(s_run):
                s_run.wait_event(ev_in[b])
                s_run.wait_event(ev_out[b])         # the previous result of this set has been read back
                sets[b]["launch"](s_run.cuda_stream)
                if world > 1 and amax_t is not None:
                    dist.all_reduce(amax_t, op=dist.ReduceOp.MAX)
                ev_run[b].record(s_run)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_run[b])
                for h, d in zip(host_out, sets[b]["outs"]):
                    h.copy_(d, non_blocking=True)
                ev_out[b].record(s_out)

        def e2e_join():
            for st in (s_in, s_run, s_out):
                stream.wait_stream(st)

        ksteps = max(4, min(args.steps, 10))
        for st in (s_in, s_run, s_out):
            st.wait_stream(stream)
        for i in range(2):
            e2e_step(i)
        e2e_join()
        barrier()
        e0.record(stream)
        for st in (s_in, s_run, s_out):
            st.wait_stream(stream)
        for i in range(ksteps):
            e2e_step(i)
        e2e_join()
        e1.record(stream)
        barrier()
        ems = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ems], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ems = float(t.item())
        e2e = {"value": w.units * world / (ems / ksteps * 1e-3) / scale_div, "unit": unit, "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "ms_per_step": ems / ksteps, "steps": ksteps,
               "pipeline": "2 buffer sets, upload / kernel / read-back on separate streams"}

    if sampler.is_alive():       # clocks were sampled through both timed regions (device-resident and end-to-end)
        sampler.stop_flag = True
        sampler.join()

    def finish():
        """Leave without tearing NCCL down: destroying the process group while an instantiated CUDA graph
        still holds captured collectives has hung at exit; every rank meets once more and exits."""
        sys.stdout.flush()
        sys.stderr.flush()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
            os._exit(0)

    if rank != 0:
        finish()
        return

    pk = peaks()
    if is_flops:
        fp8 = name != "c4"
        peak = pk["bf16_tflops"] * (2.0 if fp8 else 1.0)
        roof = {"bound": "tensor", "achieved": w.units / (ms_per_step * 1e-3) / 1e12, "peak": peak, "unit": "TFLOP/s",
                "peak_source": f"{pk['source']}: " + ("2 x bf16_tflops burst (FP8 issues at twice the BF16 rate)" if fp8 else "bf16_tflops burst"),
                "nominal_peak": 4500.0 if fp8 else 2250.0}
    else:
        roof = {"bound": "hbm", "achieved": w.units / (ms_per_step * 1e-3) / 1e9, "peak": pk["hbm_gbs"], "unit": "GB/s",
                "peak_source": f"{pk['source']}: hbm_gbs (copy)", "nominal_peak": 8000.0}
    roof["frac"] = roof["achieved"] / roof["peak"]
    roof["frac_of_nominal"] = roof["achieved"] / roof["nominal_peak"]
    roof["traffic"] = NCU_TRAFFIC_BYTES.get(name)
    roof["algorithmic_units_per_launch"] = w.units
    roof["kernel_ms"] = ms_per_step

    cpu = None
    if world == 1 and not args.no_cpu:
        import oracle as orc
        v, u, sample, _ = cpu_sample(name)
        cpu = {"value": v, "unit": u, "cores": orc.threads(), "kind": "port", "sample": sample}
        if w.kind == "gemm":
            cpu["parity_sample"] = parity_sample(w, orc)

    if reduce_amax:
        config["settle_steps_untimed"] = settle_steps
        config["amax_reduce"] = {
            "fused": "every step writes its amax into its own slot; one max-all-reduce over the slots after the last "
                     "step, inside the timed region",
            "inline": "one max-all-reduce of one float after every step", "overlap": "the reduction of step i runs "
            "beside step i + 1"}[mode]
        if inline_aux is not None:
            config["with_one_all_reduce_per_step"] = {"ms_per_step": inline_aux,
                                                      "value": w.units * world / (inline_aux * 1e-3) / scale_div}
    line = {"metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": {"c1": "fp8 (e5m2 x e5m2, f32 accumulate)", "c2": "fp8 (e5m2 x e4m3, f32 accumulate)",
                      "c4": "bf16 (e5m2 widened exactly, f32 accumulate)"}.get(name, "f32"),
            "data": "synthetic", "config": config, "clocks": sampler.summary(), "e2e": e2e,
            "gpu_launches": args.steps * w.launches_per_pass, "timed_as": "cuda_graph" if graph is not None else "stream", "roofline": roof, "cpu_baseline": cpu,
            "tolerance": "GEMM/GEMV: 1 ulp of the output format + k * 2^-23 * sum|a*b|*|s| (checked by tests/ on every "
                         "output of the small cases and on sampled rows/columns at full size); casts, AdamW: bit-exact",
            "gemm_fault": fault}
    print(json.dumps(line), flush=True)
    finish()


if __name__ == "__main__":
    main()
