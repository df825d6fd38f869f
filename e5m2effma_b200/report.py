"""Turns bench.py JSON lines into the markdown tables of the documentation -- the role bench/report.py
(lines 88-162) plays for the reference, without its clock pinning.

    python -m e5m2effma_b200.report FILE [FILE ...]     # files holding one bench.py line each (N = 1, 2, 4, 8 ...)
    python -m e5m2effma_b200.report --run               # runs `python bench.py` (one GPU) first and reports that

One table per line: for N = 1 every workload of the run (headline first) with time, value, roofline fractions in
the burst and the sustained regime, clocks and the observed error; for N > 1 the strong-scaling figures of every
workload (kernel only, with NCCL collectives, with the fused epilogue broadcast).  A line that carries `gemm_rows`
(the layout and pairing rows of the reference's GEMM benchmark) gets a third table.
"""
import argparse
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def load(path):
    lines = [l for l in open(path) if l.startswith("{")]
    if not lines:
        raise SystemExit(f"{path}: no JSON line")
    return json.loads(lines[-1])


def _pct(x):
    return "-" if x is None else f"{100 * x:.1f} %"


def _err(e):
    if not e:
        return "-"
    parts = []
    if "accumulation" in e:
        parts.append(f"{e['accumulation']['max_error_in_units_of_2^-23_sum_abs_products']:.2f} x 2^-23 sum|ab| (FP32 out)")
    if "output" in e:
        parts.append(f"{e['output']['max_error_in_output_ulps']:.3f} ulp ({e['output']['output']} out)")
    return ", ".join(parts) or "-"


def single_gpu_table(d):
    rows = ["| workload | time / step | value | of measured peak | of nominal | sustained: time, of sustained peak, SM MHz | SM MHz (burst), reasons | observed error |",
            "|---|---|---|---|---|---|---|---|"]

    def row(name, e, err):
        r = e["roofline"]
        s = r.get("sustained")
        sus = "-" if not s else f"{s['ms_per_step'] * 1e3:.1f} us, {_pct(s['frac'])}, {s['clocks'].get('sm_mhz')}"
        c = e.get("clocks") or {}
        return (f"| {name} | {e['ms_per_step'] * 1e3:.1f} us | {e['value']:.0f} {e['unit']} | {_pct(r['frac'])} | {_pct(r['frac_of_nominal'])} | {sus} | "
                f"{c.get('sm_mhz')} {','.join(c.get('reasons', [])) or '-'} | {_err(err)} |")

    rows.append(row(d["config"]["workload"], d, (d.get("cpu_baseline") or {}).get("observed_error")))
    for name, e in (d.get("workloads") or {}).items():
        rows.append(f"| {name} | failed: {e['error']} | | | | | | |" if "error" in e else row(e["workload"], e, e.get("observed_error")))
    out = "\n".join(rows) + "\n"
    if d.get("e2e"):
        e = d["e2e"]
        out += (f"\nEnd to end (host buffers, copies inside the timed region): {e['ms_per_step']:.2f} ms per step = {e['value']:.0f} {e['unit']}; "
                f"{e['h2d_bytes_per_step'] / 1e6:.1f} MB up, {e['d2h_bytes_per_step'] / 1e6:.1f} MB down per step.\n")
    if d.get("cpu_baseline"):
        c = d["cpu_baseline"]
        out += f"CPU oracle ({c['cores']} threads, {c['kind']}): {c['value']:.3f} {c['unit']} on {c['sample']}.\n"
    return out


def rows_table(d):
    """The layout / pairing rows of the reference's GEMM benchmark (bench/bench_gemm.cu:33-70, M = N = K = 4096) and
    the rows of its GEMV benchmark (bench/bench_gemv.cu:38-47, 8192 x 8192 weights)."""
    rows = ["| row | time | value | kernel | of that unit's peak | SM MHz |", "|---|---|---|---|---|---|"]
    for r in d.get("gemm_rows") or []:
        if "error" in r:
            rows.append(f"| {r['row']} | failed: {r['error']} | | | | |")
        else:
            rows.append(f"| {r['row']} | {r['ms_per_step'] * 1e3:.1f} us | {r['value']:.0f} {r['unit']} | {r['kernel']} | "
                        f"{_pct(r['frac'])} of {r['peak']:.0f} ({r['peak_source']}) | {(r.get('clocks') or {}).get('sm_mhz')} |")
    return "\n".join(rows) + "\n"


def strong_table(d):
    n = d["n_gpus"]
    rows = [f"| workload (N = {n}) | T1 (one GPU, full problem) | kernel only: time, T1/(N T) | NCCL collectives: time, T1/(N T) | fused epilogue broadcast: time, T1/(N T) |",
            "|---|---|---|---|---|"]

    def cell(x):
        if not x:
            return "-"
        if "unavailable" in x:
            return "unavailable"
        return f"{x['ms_per_step'] * 1e3:.1f} us, {_pct(x['strong_efficiency'])}"

    def row(name, s):
        return (f"| {name} | {s['full_problem_one_gpu_ms'] * 1e3:.1f} us | {cell(s.get('kernel_only'))} | {cell(s.get('with_collectives_nccl'))} | "
                f"{cell(s.get('with_collectives_fused'))} |")

    rows.append(row(d["config"]["workload"], d["strong_scaling"]))
    for name, e in (d.get("workloads") or {}).items():
        if "strong_scaling" in e:
            rows.append(row(e["workload"], e["strong_scaling"]))
    out = "\n".join(rows) + "\n"
    if d.get("e2e"):
        e = d["e2e"]
        out += (f"\nEnd to end at N = {n}: {e['ms_per_step']:.2f} ms per step = {e['value']:.0f} {e['unit']}; per rank "
                f"{e.get('h2d_bytes_per_step_per_rank', 0) / 1e6:.1f} MB up, {e.get('d2h_bytes_per_step_per_rank', 0) / 1e6:.1f} MB down.\n")
    w = d.get("weak_scaling") or (d["config"].get("weak") if isinstance(d["config"].get("weak"), dict) else None)
    if w:
        out += f"Weak scaling (every rank the full problem, amax reduced every step): {w['ms_per_step'] * 1e3:.1f} us per step, {w['value']:.0f} {w['unit']}.\n"
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("files", nargs="*")
    ap.add_argument("--run", action="store_true", help="run bench.py on one GPU first and report its line")
    args = ap.parse_args()
    lines = [load(f) for f in args.files]
    if args.run:
        out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py")], capture_output=True, text=True)
        if out.returncode != 0:
            raise SystemExit(out.stderr[-2000:])
        lines.append(json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][-1]))
    for d in lines:
        print(single_gpu_table(d) if d["n_gpus"] == 1 else strong_table(d))
        if d.get("gemm_rows"):
            print(rows_table(d))


if __name__ == "__main__":
    main()
