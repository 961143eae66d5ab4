"""Benchmark harness: scenario matrix -> one training subprocess per experiment -> summary table.

Counterpart of the reference's scripts/benchmarks/benchmark.py:429-1119.  What it keeps: the YAML inputs
(``scenarios*.yaml`` with a ``scenarios`` list of ``{name, framework_config: [...], arguments: {...}}`` and
``defaults.yaml``), the experiment matrix (scenario x model x framework config x number of GPUs x effective batch
size), one directory per experiment holding ``stdout`` / ``stderr`` / ``command.sh`` / ``script.json`` /
``results.json``, framework configs looked up by short name in ``sample-configurations/CONTENTS.yaml`` and handed
over in ``ACCELERATION_FRAMEWORK_CONFIG_FILE``, an optional ``nvidia-smi`` memory logger, traceback extraction,
re-runs that skip finished experiments, and the final ``raw_summary.csv``.  What differs: experiments launch this
repository's own trainer (``benchmarks/sft_trainer.py``), multi-GPU runs go through ``torch.distributed.run`` on
127.0.0.1 with one rank per GPU, and every list-valued argument (not only the model name) spans the matrix.
"""
from __future__ import annotations

import argparse
import ast
import csv
import itertools
import json
import os
import re
import shlex
import subprocess
import sys
import time
from dataclasses import dataclass, field
from typing import Any, Dict, Iterable, List, Optional

import yaml

HERE = os.path.dirname(os.path.abspath(__file__))
REPO_ROOT = os.path.abspath(os.path.join(HERE, "..", ".."))
SAMPLE_CONFIG_DIR = os.path.join(REPO_ROOT, "sample-configurations")
TRAINER_MODULE = "fms_acceleration_b200.benchmarks.sft_trainer"
ENV_CONFIG = "ACCELERATION_FRAMEWORK_CONFIG_FILE"

FILE_STDOUT, FILE_STDERR = "stdout", "stderr"
FILE_RESULTS, FILE_COMMAND, FILE_ARGS = "results.json", "command.sh", "script.json"
FILE_SUMMARY, FILE_MEM = "raw_summary.csv", "gpu_memory_logs.csv"
DIR_PREFIX = "exp"

# arguments whose list value is ONE value (everything else that is a list spans the matrix)
LIST_VALUED_ARGUMENTS = ("target_modules", "padding_free")
TRACEBACK_START = re.compile(r"Traceback \(most recent call last\)")
TRACEBACK_END = re.compile(r"^\w+(\.\w+)*(Error|Exception)\b")
IGNORED_TRACEBACKS = ("torch.distributed.elastic.multiprocessing.errors.ChildFailedError",)


# --------------------------------------------------------------------------------------- inputs
def framework_config_files(contents_path: Optional[str] = None) -> Dict[str, str]:
    """short name -> absolute path, from the generated table of contents."""
    contents_path = contents_path or os.path.join(SAMPLE_CONFIG_DIR, "CONTENTS.yaml")
    with open(contents_path, encoding="utf-8") as fh:
        rows = yaml.safe_load(fh)["framework_configs"]
    base = os.path.dirname(contents_path)
    return {r["shortname"]: os.path.join(base, r["filename"]) for r in rows}


@dataclass
class Scenario:
    name: str
    framework_configs: List[Optional[str]]
    arguments: Dict[str, Any]
    slow: bool = False  # a slow scenario runs only when it is asked for by name

    def argument_sets(self) -> Iterable[Dict[str, Any]]:
        """Cartesian product over the list-valued arguments."""
        keys = [k for k, v in self.arguments.items() if isinstance(v, list) and k not in LIST_VALUED_ARGUMENTS]
        fixed = {k: v for k, v in self.arguments.items() if k not in keys}
        for combo in itertools.product(*(self.arguments[k] for k in keys)):
            out = dict(fixed)
            out.update(dict(zip(keys, combo)))
            yield out


def load_scenarios(path: str, only: Optional[List[str]] = None) -> List[Scenario]:
    with open(path, encoding="utf-8") as fh:
        doc = yaml.safe_load(fh)
    out = []
    for s in doc["scenarios"]:
        if only and s["name"] not in only:
            continue
        if not only and s.get("slow"):
            # unfiltered runs leave out the scenarios marked slow (scripts/benchmarks/benchmark.py:722-728)
            print(f"skipping slow scenario {s['name']!r}: name it to run it", file=sys.stderr)
            continue
        fcs = s.get("framework_config") or [None]
        out.append(Scenario(s["name"], list(fcs), dict(s.get("arguments") or {}), bool(s.get("slow", False))))
    return out


def load_defaults(path: Optional[str]) -> Dict[str, Any]:
    if not path:
        return {}
    with open(path, encoding="utf-8") as fh:
        return yaml.safe_load(fh) or {}


# --------------------------------------------------------------------------------------- experiments
@dataclass
class Experiment:
    number: int
    scenario: str
    framework_config: Optional[str]
    framework_config_file: Optional[str]
    num_gpus: int
    arguments: Dict[str, Any]
    root: str
    master_port: int = 29500
    result: Dict[str, Any] = field(default_factory=dict)

    @property
    def directory(self) -> str:
        return os.path.join(self.root, f"{DIR_PREFIX}_{self.number}")

    def path(self, name: str) -> str:
        return os.path.join(self.directory, name)

    # -- command line
    def argv(self) -> List[str]:
        if self.num_gpus > 1:
            cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={self.num_gpus}",
                   "--master-addr", "127.0.0.1", "--master-port", str(self.master_port), "-m", TRAINER_MODULE]
        else:
            cmd = [sys.executable, "-m", TRAINER_MODULE]
        for k, v in self.arguments.items():
            if v is None:
                continue
            # the launcher's parser takes a bare ``--r`` for an abbreviation of its own options: spell it out
            cmd.append("--lora_r" if k == "r" else f"--{k}")
            if isinstance(v, (list, tuple)):
                cmd.extend(str(x) for x in v)
            else:
                cmd.append(str(v))
        return cmd

    def environment(self) -> Dict[str, str]:
        env = {"CUDA_VISIBLE_DEVICES": ",".join(str(i) for i in range(self.num_gpus))}
        if self.framework_config_file:
            env[ENV_CONFIG] = self.framework_config_file
        return env

    def shell_command(self) -> str:
        env = " ".join(f"{k}={shlex.quote(v)}" for k, v in self.environment().items())
        return f"{env} {' '.join(shlex.quote(a) for a in self.argv())}"

    # -- state on disk
    def is_completed(self) -> bool:
        try:
            with open(self.path(FILE_RESULTS), encoding="utf-8") as fh:
                res = json.load(fh)
        except (OSError, ValueError):
            return False
        return not res.get("error_messages") and "train_runtime" in res

    def write_description(self) -> None:
        os.makedirs(self.directory, exist_ok=True)
        with open(self.path(FILE_COMMAND), "w", encoding="utf-8") as fh:
            fh.write("#!/bin/sh\n" + self.shell_command() + "\n")
        with open(self.path(FILE_ARGS), "w", encoding="utf-8") as fh:
            json.dump({"scenario": self.scenario, "framework_config": self.framework_config, "num_gpus": self.num_gpus,
                       "arguments": self.arguments, "acceleration_framework_config_file": self.framework_config_file},
                      fh, indent=2)

    # -- execution
    def run(self, dry_run: bool = False, log_memory: bool = False, timeout: Optional[float] = None) -> Dict[str, Any]:
        self.write_description()
        if dry_run:
            self.result = {"error_messages": ["dry_run"]}
            return self.result
        env = dict(os.environ)
        env.update(self.environment())
        env["PYTHONPATH"] = REPO_ROOT + os.pathsep + env.get("PYTHONPATH", "")
        logger = None
        if log_memory:
            logger = start_memory_logger(self.path(FILE_MEM), range(self.num_gpus))
        t0 = time.time()
        with open(self.path(FILE_STDOUT), "w") as so, open(self.path(FILE_STDERR), "w") as se:
            try:
                rc = subprocess.run(self.argv(), stdout=so, stderr=se, env=env, cwd=REPO_ROOT, timeout=timeout).returncode
            except subprocess.TimeoutExpired:
                rc = -9
        if logger is not None:
            stop_memory_logger(logger)
        res = parse_stdout(self.path(FILE_STDOUT))
        errors = extract_tracebacks(self.path(FILE_STDERR))
        if rc != 0 and not errors:
            errors = [f"exit code {rc}"]
        if errors:
            res["error_messages"] = errors
        res["wall_clock_s"] = round(time.time() - t0, 2)
        if log_memory:
            res.update(memory_metrics(self.path(FILE_MEM)))
        with open(self.path(FILE_RESULTS), "w", encoding="utf-8") as fh:
            json.dump(res, fh, indent=2)
        self.result = res
        return res

    def summary_row(self) -> Dict[str, Any]:
        row = {"experiment": self.number, "scenario": self.scenario, "framework_config": self.framework_config or "none",
               "num_gpus": self.num_gpus, "acceleration_framework_config_file": self.framework_config_file}
        row.update({k: (" ".join(map(str, v)) if isinstance(v, (list, tuple)) else v) for k, v in self.arguments.items()})
        res = dict(self.result)
        if "error_messages" in res:
            res["error_messages"] = " | ".join(m.strip().splitlines()[-1] for m in res["error_messages"] if m.strip())
        row.update(res)
        return row


# --------------------------------------------------------------------------------------- output parsing
def parse_stdout(path: str) -> Dict[str, Any]:
    """Final metrics = the last dict-like line that has ``train_runtime``; the per-step dicts before it give the
    loss trace (reference: scripts/benchmarks/benchmark.py:539-568 keeps only the last dict)."""
    final: Dict[str, Any] = {}
    trace: List[float] = []
    try:
        with open(path, encoding="utf-8", errors="replace") as fh:
            for line in fh:
                line = line.strip()
                if not (line.startswith("{") and line.endswith("}")):
                    continue
                try:
                    d = ast.literal_eval(line)
                except (ValueError, SyntaxError):
                    try:
                        d = json.loads(line)
                    except ValueError:
                        continue
                if not isinstance(d, dict):
                    continue
                if "train_runtime" in d:
                    final = d
                elif "loss" in d:
                    trace.append(float(d["loss"]))
    except OSError:
        pass
    if trace:
        final = dict(final)
        final["loss_trace"] = trace
    return final


def extract_tracebacks(path: str) -> List[str]:
    out: List[str] = []
    cur: Optional[List[str]] = None
    try:
        with open(path, encoding="utf-8", errors="replace") as fh:
            for line in fh:
                if TRACEBACK_START.search(line):
                    cur = [line]
                    continue
                if cur is not None:
                    cur.append(line)
                    if TRACEBACK_END.match(line.strip()):
                        text = "".join(cur)
                        if not any(p in text for p in IGNORED_TRACEBACKS):
                            out.append(text)
                        cur = None
    except OSError:
        pass
    return out


def start_memory_logger(path: str, gpus: Iterable[int]):
    """``nvidia-smi`` sampling ``memory.used`` once per second into a CSV (a read-only query)."""
    try:
        fh = open(path, "w")
        proc = subprocess.Popen(["nvidia-smi", "--query-gpu=timestamp,name,index,memory.used", "--format=csv",
                                 "-l", "1", "-i", ",".join(map(str, gpus))], stdout=fh, stderr=subprocess.DEVNULL)
        return proc, fh
    except OSError:
        return None


def stop_memory_logger(handle) -> None:
    if handle is None:
        return
    proc, fh = handle
    proc.terminate()
    try:
        proc.wait(timeout=5)
    except subprocess.TimeoutExpired:
        proc.kill()
    fh.close()


def memory_metrics(path: str) -> Dict[str, Any]:
    """Peak ``memory.used`` per GPU, averaged over the GPUs, in MiB."""
    peaks: Dict[str, float] = {}
    name = None
    try:
        with open(path, encoding="utf-8") as fh:
            rd = csv.reader(fh)
            header = [h.strip() for h in next(rd)]
            i_idx, i_mem, i_name = header.index("index"), header.index("memory.used [MiB]"), header.index("name")
            for row in rd:
                if len(row) <= i_mem:
                    continue
                used = float(row[i_mem].replace("MiB", "").strip())
                peaks[row[i_idx].strip()] = max(peaks.get(row[i_idx].strip(), 0.0), used)
                name = row[i_name].strip()
    except (OSError, StopIteration, ValueError):
        return {}
    if not peaks:
        return {}
    return {"mem_nvidia_mem_reserved": sum(peaks.values()) / len(peaks), "gpu_device_name": name}


# --------------------------------------------------------------------------------------- matrix
def build_experiments(scenarios: List[Scenario], defaults: Dict[str, Any], num_gpus: List[int],
                      effective_batch_sizes: List[int], root: str, config_files: Dict[str, str],
                      extra: Optional[Dict[str, Any]] = None, base_port: int = 29511,
                      matrices: Optional[Dict[str, List[Any]]] = None) -> List[Experiment]:
    """``matrices``: further run-wide dimensions (argument name -> values, e.g. ``max_seq_length``, ``packing``) that
    multiply every scenario like the numbers of GPUs and the effective batch sizes do."""
    exps: List[Experiment] = []
    n = 0
    dims = {k: v for k, v in (matrices or {}).items() if v}
    combos = [dict(zip(dims, c)) for c in itertools.product(*dims.values())] or [{}]
    for sc in scenarios:
        for base_args, combo in itertools.product(list(sc.argument_sets()), combos):
            args = {**combo, **base_args}  # what a scenario fixes is not varied
            for fc in sc.framework_configs:
                if fc is not None and fc not in config_files:
                    # a short name without a sample configuration drops out of the matrix, as in the reference
                    # (scripts/benchmarks/benchmark.py:388-403; its own scenarios-granite.yaml names one)
                    print(f"scenario {sc.name!r}: no sample configuration named {fc!r}, skipped", file=sys.stderr)
                    continue
                for g, ebs in itertools.product(num_gpus, effective_batch_sizes):
                    merged = dict(defaults)
                    merged.update(args)
                    merged.update(extra or {})
                    accum = merged.get("gradient_accumulation_steps") or 1
                    if "per_device_train_batch_size" not in args:
                        if ebs % (g * accum) != 0:
                            continue  # this effective batch size cannot be split evenly
                        merged["per_device_train_batch_size"] = ebs // (g * accum)
                    exps.append(Experiment(n, sc.name, fc, config_files.get(fc) if fc else None, g, merged, root,
                                           master_port=base_port + n % 400))
                    n += 1
    return exps


def write_summary(exps: List[Experiment], path: str) -> None:
    rows = [e.summary_row() for e in exps]
    cols: List[str] = []
    for r in rows:
        for k in r:
            if k not in cols and k != "loss_trace":
                cols.append(k)
    with open(path, "w", newline="", encoding="utf-8") as fh:
        w = csv.DictWriter(fh, fieldnames=cols, extrasaction="ignore")
        w.writeheader()
        for r in rows:
            w.writerow(r)


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(description="run the benchmark matrix")
    ap.add_argument("--num_gpus", "--num_gpus_matrix", dest="num_gpus", type=int, nargs="+", default=[1])
    ap.add_argument("--effective_batch_size_matrix", type=int, nargs="+", default=[4])
    ap.add_argument("--scenarios_config_path", default=os.path.join(HERE, "scenarios.yaml"))
    ap.add_argument("--defaults_config_path", default=os.path.join(HERE, "defaults.yaml"))
    ap.add_argument("--results_output_path", default="benchmark_results")
    ap.add_argument("--run_only_scenarios", nargs="*", default=None)
    ap.add_argument("--training_data_path", default=None, help="tokenised JSON made by data_processing.py")
    ap.add_argument("--max_seq_length", type=int, default=None)
    ap.add_argument("--max_steps", type=int, default=None)
    ap.add_argument("--dry_run", action="store_true", help="write command.sh for every experiment, run nothing")
    ap.add_argument("--no_overwrite", action="store_true", help="skip experiments that already have results")
    ap.add_argument("--log_nvidia_smi", action="store_true")
    ap.add_argument("--timeout", type=float, default=None, help="seconds per experiment")
    # further options of the reference's runner (scripts/benchmarks/benchmark.py:1010-1110)
    tf = lambda v: str(v).lower() in ("1", "true", "yes")  # noqa: E731
    ap.add_argument("--max_seq_len_matrix", type=int, nargs="+", default=None, help="sequence lengths to multiply by")
    ap.add_argument("--packing_matrix", type=tf, nargs="+", default=None, help="packing settings to multiply by")
    ap.add_argument("--acceleration_framework_config_keypairs", nargs="+", default=None,
                    help="short name / file pairs that replace the sample-configuration table")
    ap.add_argument("--process_port", type=int, default=29511, help="first rendezvous port of multi-GPU experiments")
    ap.add_argument("--dataset_save_path", default=None,
                    help="directory with a tokenised cache made by data_processing.py (cache_bench.json)")
    ap.add_argument("--no_data_processing", action="store_true", help="accepted: an existing cache is always kept")
    ap.add_argument("--preload_models", action="store_true", help="resolve every model name before anything runs")
    ap.add_argument("--log_memory_hf", action="store_true", help="record the allocator's peak memory")
    ap.add_argument("--accelerate_config", default=None,
                    help="accepted for call compatibility: ranks are launched with torch.distributed.run")
    a = ap.parse_args(argv)

    extra = {k: v for k, v in (("training_data_path", a.training_data_path), ("max_seq_length", a.max_seq_length),
                               ("max_steps", a.max_steps)) if v is not None}
    if a.log_nvidia_smi or a.log_memory_hf:
        extra["skip_memory_metrics"] = False
    if a.dataset_save_path and "training_data_path" not in extra:
        cache = os.path.join(a.dataset_save_path, "cache_bench.json")
        if os.path.isfile(cache):
            extra["training_data_path"] = cache
        else:
            print(f"no tokenised cache at {cache}: experiments use synthetic packed documents", file=sys.stderr)
    config_files = framework_config_files()
    if a.acceleration_framework_config_keypairs:
        pairs = a.acceleration_framework_config_keypairs
        if len(pairs) % 2:
            ap.error("--acceleration_framework_config_keypairs takes short name / file pairs")
        config_files = dict(zip(pairs[0::2], pairs[1::2]))
    scenarios = load_scenarios(a.scenarios_config_path, a.run_only_scenarios)
    if a.preload_models:
        from ..models.builder import resolve_config

        for sc in scenarios:
            names = sc.arguments.get("model_name_or_path", [])
            for name in names if isinstance(names, list) else [names]:
                resolve_config(name)
                print(f"scenario {sc.name!r}: model {name!r} resolves")
    matrices = {"max_seq_length": a.max_seq_len_matrix, "packing": a.packing_matrix}
    exps = build_experiments(scenarios, load_defaults(a.defaults_config_path), a.num_gpus,
                             a.effective_batch_size_matrix, a.results_output_path, config_files, extra,
                             base_port=a.process_port, matrices=matrices)
    os.makedirs(a.results_output_path, exist_ok=True)
    print(f"{len(exps)} experiments from {len(scenarios)} scenarios")
    for e in exps:
        if a.no_overwrite and e.is_completed():
            with open(e.path(FILE_RESULTS), encoding="utf-8") as fh:
                e.result = json.load(fh)
            print(f"[{e.number}] {e.scenario} / {e.framework_config}: kept")
            continue
        res = e.run(dry_run=a.dry_run, log_memory=a.log_nvidia_smi, timeout=a.timeout)
        status = "dry run" if a.dry_run else ("FAILED" if res.get("error_messages") else
                                              f"{res.get('train_tokens_per_second', '?')} tokens/s/GPU")
        print(f"[{e.number}] {e.scenario} / {e.framework_config} / {e.arguments.get('model_name_or_path')} "
              f"x{e.num_gpus}: {status}", flush=True)
    write_summary(exps, os.path.join(a.results_output_path, FILE_SUMMARY))
    return 0


if __name__ == "__main__":
    sys.exit(main())
