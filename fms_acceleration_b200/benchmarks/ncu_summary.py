"""Condense the raw CSV page of an Nsight Compute report into the handful of figures a roofline summary needs.

    ncu -i report.ncu-rep --page raw --csv > raw.csv
    python -m fms_acceleration_b200.benchmarks.ncu_summary raw.csv [--kernel regex] [--flops F] [--bytes B]

Prints one markdown table row group per captured launch: duration, DRAM bytes read/written and throughput, tensor
pipe utilisation, achieved occupancy (active warps), registers per thread, dynamic shared memory, and the top warp
stall reasons.  With ``--flops`` / ``--bytes`` (algorithmic work per launch) the achieved rate and the fraction of
the measured peaks are added.  Reads the CSV only; it never runs a profiler.
"""
from __future__ import annotations

import argparse
import csv
import re
import sys
from typing import Dict, List, Optional

from ..utils.profiling import measured_peaks

WANTED = {
    "gpu__time_duration.sum": "duration",
    "dram__bytes_read.sum": "dram read",
    "dram__bytes_write.sum": "dram write",
    "gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed": "dram throughput %",
    "sm__pipe_tensor_cycles_active.avg.pct_of_peak_sustained_active": "tensor pipe active %",
    "sm__pipe_tensor_subpipe_hmma_cycles_active.avg.pct_of_peak_sustained_active": "tensor (hmma) active %",
    "sm__warps_active.avg.pct_of_peak_sustained_active": "active warps %",
    "sm__throughput.avg.pct_of_peak_sustained_elapsed": "sm throughput %",
    "lts__t_sector_hit_rate.pct": "L2 hit rate %",
    "launch__registers_per_thread": "registers/thread",
    "launch__shared_mem_per_block_dynamic": "dynamic smem/block",
    "launch__grid_size": "grid",
    "launch__block_size": "block",
}


def parse(path: str) -> List[Dict[str, str]]:
    with open(path, newline="", encoding="utf-8", errors="replace") as fh:
        lines = [l for l in fh if l.startswith('"')]
    rows = list(csv.reader(lines))
    if len(rows) < 3:
        return []
    header, units, data = rows[0], rows[1], rows[2:]
    out = []
    for r in data:
        d = {}
        for h, u, v in zip(header, units, r):
            d[h] = v
            d[h + "::unit"] = u
        out.append(d)
    return out


def _num(s: str) -> Optional[float]:
    try:
        return float(s.replace(",", ""))
    except (ValueError, AttributeError):
        return None


def to_seconds(v: float, unit: str) -> float:
    return v * {"ns": 1e-9, "us": 1e-6, "ms": 1e-3, "s": 1.0, "nsecond": 1e-9, "usecond": 1e-6, "msecond": 1e-3,
                "second": 1.0}.get(unit, 1e-9)


def to_bytes(v: float, unit: str) -> float:
    return v * {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9, "Tbyte": 1e12}.get(unit, 1.0)


def summarise(rows: List[Dict[str, str]], kernel: Optional[str], flops: float, nbytes: float) -> str:
    pk = measured_peaks()
    out = []
    for r in rows:
        name = r.get("Kernel Name", "?")
        if kernel and not re.search(kernel, name):
            continue
        out.append(f"### {name}  (launch id {r.get('ID', '?')})\n")
        out.append("| metric | value |\n|---|---|")
        dur = None
        dram = 0.0
        for key, label in WANTED.items():
            if key not in r:
                continue
            v, unit = _num(r[key]), r.get(key + "::unit", "")
            if v is None:
                continue
            if key == "gpu__time_duration.sum":
                dur = to_seconds(v, unit)
                out.append(f"| {label} | {dur * 1e3:.4f} ms |")
            elif key.startswith("dram__bytes"):
                b = to_bytes(v, unit)
                dram += b
                out.append(f"| {label} | {b / 1e6:.1f} MB |")
            else:
                out.append(f"| {label} | {v:g} {unit} |")
        stalls = sorted(((k, _num(v)) for k, v in r.items()
                         if k.startswith("smsp__average_warps_issue_stalled") and k.endswith("_per_issue_active.ratio")
                         and _num(v) is not None), key=lambda kv: -kv[1])[:4]
        for k, v in stalls:
            short = k.replace("smsp__average_warps_issue_stalled_", "").replace("_per_issue_active.ratio", "")
            out.append(f"| stall: {short} | {v:.2f} warps/issue |")
        if dur:
            out.append(f"| dram traffic / time | {dram / dur / 1e9:.0f} GB/s = {dram / dur / 1e9 / pk['hbm_gbs']:.2f} of "
                       f"{pk['source']} copy bandwidth |")
            if flops:
                tf = flops / dur / 1e12
                out.append(f"| algorithmic FLOP rate | {tf:.0f} TFLOP/s = {tf / pk['bf16_tflops']:.2f} of {pk['source']} "
                           f"cuBLAS bf16 |")
            if nbytes:
                gb = nbytes / dur / 1e9
                out.append(f"| algorithmic byte rate | {gb:.0f} GB/s = {gb / pk['hbm_gbs']:.2f} of {pk['source']} copy "
                           f"bandwidth |")
        out.append("")
    return "\n".join(out)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("csv")
    ap.add_argument("--kernel", default=None)
    ap.add_argument("--flops", type=float, default=0.0)
    ap.add_argument("--bytes", type=float, default=0.0)
    a = ap.parse_args(argv)
    rows = parse(a.csv)
    if not rows:
        print("no launches found in the CSV", file=sys.stderr)
        return 1
    print(summarise(rows, a.kernel, a.flops, a.bytes))
    return 0


if __name__ == "__main__":
    sys.exit(main())
