"""Gather the per-experiment results of a benchmark run into one CSV.

    python -m fms_acceleration_b200.benchmarks.display_bench_results RESULT_DIR [--result_file benchmarks.csv]
        [--keep_columns a b ...] [--remove_columns c d ...]

Reads every ``exp_*/script.json`` + ``results.json`` below ``RESULT_DIR`` (reference:
scripts/benchmarks/display_bench_results.py:10-53).  Argument columns that have the same value in every experiment
are dropped unless listed in ``--keep_columns``; ``--remove_columns`` drops columns unconditionally; experiments that
failed are listed on stderr and left out of the table.
"""
from __future__ import annotations

import argparse
import csv
import json
import os
import sys
from typing import Any, Dict, List, Optional


def gather(result_dir: str):
    rows, failed = [], []
    for name in sorted(os.listdir(result_dir), key=lambda s: (len(s), s)):
        d = os.path.join(result_dir, name)
        if not (name.startswith("exp_") and os.path.isdir(d)):
            continue
        try:
            with open(os.path.join(d, "script.json"), encoding="utf-8") as fh:
                script = json.load(fh)
            with open(os.path.join(d, "results.json"), encoding="utf-8") as fh:
                res = json.load(fh)
        except (OSError, ValueError):
            failed.append((name, "no results"))
            continue
        if res.get("error_messages"):
            failed.append((name, str(res["error_messages"][-1]).strip().splitlines()[-1]))
            continue
        row: Dict[str, Any] = {"scenario": script["scenario"], "framework_config": script["framework_config"] or "none",
                               "num_gpus": script["num_gpus"]}
        for k, v in script["arguments"].items():
            row[k] = " ".join(map(str, v)) if isinstance(v, list) else v
        row.update({k: v for k, v in res.items() if k != "loss_trace"})
        rows.append(row)
    return rows, failed


def select_columns(rows: List[Dict[str, Any]], argument_columns: List[str], keep: List[str], remove: List[str]) -> List[str]:
    cols: List[str] = []
    for r in rows:
        for k in r:
            if k not in cols:
                cols.append(k)
    out = []
    for c in cols:
        if c in remove:
            continue
        if c in argument_columns and c not in keep:
            values = {json.dumps(r.get(c), sort_keys=True) for r in rows}
            if len(values) <= 1:
                continue  # the same everywhere: carries no information
        out.append(c)
    return out


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("result_dir", nargs="+", help="one or more result directories (their experiments are pooled)")
    ap.add_argument("--result_file", default=None)
    ap.add_argument("--keep_columns", nargs="*", default=[])
    ap.add_argument("--remove_columns", nargs="*", default=[])
    a = ap.parse_args(argv)
    rows, failed = [], []
    for d in a.result_dir:
        r, f = gather(d)
        rows += r
        failed += [(os.path.join(d, name), why) for name, why in f]
    for name, why in failed:
        print(f"{name}: {why}", file=sys.stderr)
    if not rows:
        print("no successful experiments", file=sys.stderr)
        return 1
    arg_cols = set()
    for d in a.result_dir:
        for name in os.listdir(d):
            p = os.path.join(d, name, "script.json")
            if os.path.exists(p):
                with open(p, encoding="utf-8") as fh:
                    arg_cols |= set(json.load(fh)["arguments"])
    cols = select_columns(rows, sorted(arg_cols), a.keep_columns, a.remove_columns)
    out = a.result_file or os.path.join(a.result_dir[0], "benchmarks.csv")
    with open(out, "w", newline="", encoding="utf-8") as fh:
        w = csv.DictWriter(fh, fieldnames=cols, extrasaction="ignore")
        w.writeheader()
        w.writerows(rows)
    print(f"{len(rows)} experiments -> {out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
