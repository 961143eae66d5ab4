"""Regression check of a benchmark table against an earlier one.

    python -m fms_acceleration_b200.benchmarks.compare_with_reference --result_dir RESULT_DIR \
        --reference_benchmark_filepath old.csv [--threshold_ratio 0.1] \
        [--indices framework_config model_name_or_path num_gpus per_device_train_batch_size] \
        [--plot_columns train_tokens_per_second train_loss mem_nvidia_mem_reserved]

Merges ``RESULT_DIR/benchmarks.csv`` with the reference table on the index columns and flags every metric whose
relative difference exceeds the threshold (reference: scripts/benchmarks/compare_with_reference.py:11-158, which
also draws scatter plots; here the comparison is written as ``comparison.csv`` and ``outliers.csv`` - plotting
needs matplotlib, which is used only when importable).  Exit code 1 when outliers exist.
"""
from __future__ import annotations

import argparse
import os
import sys
from typing import List, Optional

import pandas as pd

DEFAULT_INDICES = ["framework_config", "peft_method", "model_name_or_path", "num_gpus", "per_device_train_batch_size"]
DEFAULT_PLOT_COLUMNS = ["mem_torch_mem_alloc_in_bytes", "mem_peak_torch_mem_alloc_in_bytes", "train_loss",
                        "train_tokens_per_second"]


def compare(new: pd.DataFrame, ref: pd.DataFrame, indices: List[str], columns: List[str], threshold: float):
    idx = [c for c in indices if c in new.columns and c in ref.columns]
    if not idx:
        raise ValueError("no index column is present in both tables")
    new, ref = new.copy(), ref.copy()
    for c in idx:
        new[c] = new[c].astype(str).fillna("none")
        ref[c] = ref[c].astype(str).fillna("none")
    merged = new.merge(ref, on=idx, how="inner", suffixes=("_new", "_ref"))
    records = []
    for col in columns:
        a, b = f"{col}_new", f"{col}_ref"
        if a not in merged.columns or b not in merged.columns:
            continue
        for _, row in merged.iterrows():
            x, y = pd.to_numeric(row[a], errors="coerce"), pd.to_numeric(row[b], errors="coerce")
            if pd.isna(x) or pd.isna(y) or y == 0:
                continue
            ratio = float(x) / float(y)
            rec = {c: row[c] for c in idx}
            rec.update({"metric": col, "new": float(x), "reference": float(y), "ratio": ratio,
                        "outlier": abs(ratio - 1.0) > threshold})
            records.append(rec)
    table = pd.DataFrame.from_records(records)
    outliers = table[table["outlier"]] if len(table) else table
    return table, outliers, len(merged)


def maybe_plot(table: pd.DataFrame, out_dir: str) -> List[str]:
    try:
        import matplotlib

        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except ImportError:
        return []
    files = []
    for metric, grp in table.groupby("metric"):
        fig, ax = plt.subplots(figsize=(5, 5))
        ax.scatter(grp["reference"], grp["new"], c=["r" if o else "b" for o in grp["outlier"]])
        lim = [min(grp["reference"].min(), grp["new"].min()), max(grp["reference"].max(), grp["new"].max())]
        ax.plot(lim, lim, "k--", linewidth=0.5)
        ax.set_xlabel("reference")
        ax.set_ylabel("new")
        ax.set_title(metric)
        path = os.path.join(out_dir, f"compare-{metric}.jpg")
        fig.savefig(path)
        plt.close(fig)
        files.append(path)
    return files


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--result_dir", default="benchmark_results")
    ap.add_argument("--reference_benchmark_filepath", required=True)
    ap.add_argument("--threshold_ratio", type=float, default=0.1)
    ap.add_argument("--indices", nargs="+", default=DEFAULT_INDICES)
    ap.add_argument("--plot_columns", nargs="+", default=DEFAULT_PLOT_COLUMNS)
    a = ap.parse_args(argv)
    new = pd.read_csv(os.path.join(a.result_dir, "benchmarks.csv"))
    ref = pd.read_csv(a.reference_benchmark_filepath)
    table, outliers, n = compare(new, ref, a.indices, a.plot_columns, a.threshold_ratio)
    table.to_csv(os.path.join(a.result_dir, "comparison.csv"), index=False)
    outliers.to_csv(os.path.join(a.result_dir, "outliers.csv"), index=False)
    maybe_plot(table, a.result_dir) if len(table) else None
    print(f"{n} experiments matched, {len(table)} metric values compared, {len(outliers)} outliers "
          f"(threshold {a.threshold_ratio:.0%})")
    if len(outliers):
        print(outliers.to_string(index=False))
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
