#!/usr/bin/env python3
"""Profile the best GEMM config per shape with Nsight Compute and report how busy the
tensor pipe and DRAM were.

Same flow and flags as the reference script (gemm/test_compute_rate.py of
HugeOrca/sm120-dl): read "BEST: M,N,K config ..." lines from BEST.txt (written by
`test_gemm_cute --benchmark`), run `test_gemm_cute --profile <config> M N K <warmup>` under
`ncu --profile-from-start off -c 1` (the harness brackets exactly one launch with
cudaProfilerStart/Stop), print one row per shape.  Flags: --binary, --best-file, --func +
--shape M N K, --only MxNxK[,...], --warmup, --out-dir.

Columns: the reference's SM% and DRAM% (sm__throughput / dram__throughput, % of peak
sustained elapsed) plus what tells how well a tcgen05 kernel runs: tensor-pipe active %, DRAM bytes
moved and the launch duration, from which TFLOP/s and GB/s follow, and the two counters that
decide the clock of a tensor-bound kernel under the power cap (operand bytes delivered from L2
to the SMs, warp instructions executed).  ncu never changes the
GPU clocks here (--clock-control none).
"""

import argparse
import csv
import io
import os
import re
import subprocess
import sys
from pathlib import Path

METRICS = {
    "sm": "sm__throughput.avg.pct_of_peak_sustained_elapsed",
    "dram": "dram__throughput.avg.pct_of_peak_sustained_elapsed",
    "tensor": "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_elapsed",
    "rd": "dram__bytes_read.sum",
    "wr": "dram__bytes_write.sum",
    "ns": "gpu__time_duration.sum",
    # what decides the clock under the power cap: operand bytes L2 -> SM and instructions issued
    "l2sm": "l1tex__m_xbar2l1tex_read_bytes.sum",
    "inst": "smsp__inst_executed.sum",
}
BEST_RE = re.compile(r"^BEST:\s*(\d+),(\d+),(\d+)\s+(\S+)")


def parse_best_file(path):
    entries = []
    with open(path) as f:
        for line in f:
            m = BEST_RE.match(line.strip())
            if m:
                entries.append((int(m.group(1)), int(m.group(2)), int(m.group(3)), m.group(4)))
    return entries


def to_number(cell):
    try:
        return float(str(cell).replace(",", ""))
    except (TypeError, ValueError):
        return None


def profile(binary, config, shape, warmup, out_dir):
    M, N, K = shape
    base = str(out_dir / f"gemm__{config}__{M}x{N}x{K}")
    cmd = ["ncu", "--clock-control", "none", "--profile-from-start", "off", "-c", "1", "--metrics",
           ",".join(METRICS.values()), "-o", base, "-f", binary, "--profile", config, str(M), str(N), str(K),
           str(warmup)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError(f"ncu failed (rc={proc.returncode})")
    raw = subprocess.run(["ncu", "-i", base + ".ncu-rep", "--csv", "--page", "raw"], capture_output=True, text=True,
                         check=True).stdout
    rows = list(csv.DictReader(io.StringIO(raw)))
    units = rows[0] if rows else {}
    out = {}
    for key, metric in METRICS.items():
        value = None
        for row in rows[1:] if len(rows) > 1 else rows:
            number = to_number(row.get(metric))
            if number is not None:
                value = number
        if value is not None and key in ("rd", "wr", "l2sm"):
            unit = (units.get(metric) or "").lower()
            value *= {"byte": 1.0, "kbyte": 1e3, "mbyte": 1e6, "gbyte": 1e9}.get(unit, 1.0)
        if value is not None and key == "ns":
            unit = (units.get(metric) or "").lower()
            value *= {"ns": 1.0, "us": 1e3, "ms": 1e6, "s": 1e9, "nsecond": 1.0, "usecond": 1e3, "msecond": 1e6}.get(unit, 1.0)
        out[key] = value
    return out


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    here = Path(__file__).resolve().parent
    ap.add_argument("--binary", default=str(here / "test_gemm_cute"))
    ap.add_argument("--best-file", default=None, help="BEST.txt path (default: next to the binary)")
    ap.add_argument("--func", default=None, help="profile a single config instead of reading BEST.txt")
    ap.add_argument("--shape", nargs=3, type=int, metavar=("M", "N", "K"), help="shape for --func")
    ap.add_argument("--only", default=None, help="comma-separated MxNxK filter")
    ap.add_argument("--all", action="store_true",
                    help="profile every BEST.txt entry; by default shapes whose operands exceed --max-gb are skipped")
    ap.add_argument("--max-gb", type=float, default=1.0,
                    help="largest A+B+C footprint profiled without --all or --only (multi-metric captures replay the "
                         "kernel and save/restore device memory, so they belong on small cases)")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--out-dir", default=None, help="directory for .ncu-rep files (default: ./ncu_out)")
    args = ap.parse_args()

    binary = os.path.abspath(args.binary)
    if not os.path.exists(binary):
        ap.error(f"binary not found: {binary}")
    out_dir = Path(args.out_dir) if args.out_dir else Path.cwd() / "ncu_out"
    out_dir.mkdir(parents=True, exist_ok=True)

    if args.func:
        if not args.shape:
            ap.error("--func requires --shape M N K")
        entries = [(*args.shape, args.func)]
    else:
        best_file = args.best_file or os.path.join(os.path.dirname(binary), "BEST.txt")
        if not os.path.exists(best_file):
            ap.error(f"BEST.txt not found: {best_file}\nRun `{binary} --benchmark` first, or pass --best-file.")
        entries = parse_best_file(best_file)
    if args.only:
        keep = {tuple(int(x) for x in s.lower().split("x")) for s in args.only.split(",")}
        entries = [e for e in entries if e[:3] in keep]
    elif not args.all and not args.func:
        small = [e for e in entries if 2.0 * (e[0] * e[2] + e[1] * e[2] + e[0] * e[1]) <= args.max_gb * 1e9]
        for e in entries:
            if e not in small:
                print(f"# skipped {e[0]}x{e[1]}x{e[2]}: operands above {args.max_gb} GB (use --only or --all)")
        entries = small
    if not entries:
        ap.error("no shapes to profile")

    print(f"# binary: {binary}")
    print(f"{'shape':<22} {'config':<44} {'SM %':>7} {'DRAM %':>7} {'tensor %':>9} {'us':>9} {'TFLOP/s':>9} {'DRAM GB':>8} {'GB/s':>8} {'L2>SM GB':>9} {'Minst':>7}")
    for M, N, K, cfg in entries:
        tag = f"{M}x{N}x{K}"
        try:
            r = profile(binary, cfg, (M, N, K), args.warmup, out_dir)
        except (RuntimeError, subprocess.CalledProcessError) as exc:
            print(f"{tag:<22} {cfg:<44} {'ERR':>7} {'ERR':>7}  ({exc})")
            continue
        fmt = lambda v, f="{:.2f}": f.format(v) if v is not None else "n/a"  # noqa: E731
        us = r["ns"] / 1e3 if r["ns"] else None
        tf = 2.0 * M * N * K / (r["ns"] * 1e-9) / 1e12 if r["ns"] else None
        gb = (r["rd"] + r["wr"]) / 1e9 if r["rd"] is not None and r["wr"] is not None else None
        gbs = gb / (r["ns"] * 1e-9) if gb is not None and r["ns"] else None
        print(f"{tag:<22} {cfg:<44} {fmt(r['sm']):>7} {fmt(r['dram']):>7} {fmt(r['tensor']):>9} {fmt(us, '{:.1f}'):>9} "
              f"{fmt(tf, '{:.1f}'):>9} {fmt(gb, '{:.3f}'):>8} {fmt(gbs, '{:.0f}'):>8} "
              f"{fmt(r['l2sm'] / 1e9 if r['l2sm'] is not None else None, '{:.2f}'):>9} "
              f"{fmt(r['inst'] / 1e6 if r['inst'] is not None else None, '{:.1f}'):>7}")


if __name__ == "__main__":
    main()
