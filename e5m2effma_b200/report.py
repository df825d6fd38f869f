"""Runs bench.py over every workload and writes a markdown table of the results -- the role
bench/run_bench.sh + bench/report.py (lines 88-162) play for the reference, without its clock pinning.

    python -m e5m2effma_b200.report [--out report.md] [--steps 20] [--warmup 5]
"""
import argparse
import json
import os
import subprocess
import sys

from .workloads import NAMES

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="report.md")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--cpu", action="store_true", help="also time the CPU oracle on every workload (slow)")
    args = ap.parse_args()
    lines = ["| workload | ms / step | value | of measured peak | of nominal | end to end | clocks (MHz, reasons) |", "|---|---|---|---|---|---|---|"]
    for name in NAMES:
        cmd = [sys.executable, os.path.join(ROOT, "bench.py"), "--workload", name, "--steps", str(args.steps), "--warmup", str(args.warmup)]
        if not args.cpu:
            cmd.append("--no-cpu")
        out = subprocess.run(cmd, capture_output=True, text=True)
        if out.returncode != 0:
            lines.append(f"| {name} | failed: {out.stderr.strip().splitlines()[-1] if out.stderr.strip() else out.returncode} | | | | | |")
            continue
        d = json.loads(out.stdout.strip().splitlines()[-1])
        r, e, c = d["roofline"], d.get("e2e") or {}, d["clocks"]
        lines.append(f"| {d['config']['workload']} | {d['ms_per_step']:.4f} | {d['value']:.1f} {d['unit']} | {100 * r['frac']:.1f} % | "
                     f"{100 * r['frac_of_nominal']:.1f} % | {e.get('value', float('nan')):.1f} {d['unit']} | {c['sm_mhz']} {','.join(c['reasons']) or '-'} |")
        print(lines[-1], flush=True)
    with open(args.out, "w") as f:
        f.write("\n".join(lines) + "\n")


if __name__ == "__main__":
    main()
