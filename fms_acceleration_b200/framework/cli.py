"""Command line of the framework: ``python -m fms_acceleration.cli {install,plugins,configs,arguments}``.

Verbs as in fms_acceleration/cli.py:36-213 of the reference.  All plugins ship in-tree here, so ``install`` only
reports that (and can build the native library); ``plugins`` lists the plugins and whether they import;
``configs`` lists the sample configurations from ``sample-configurations/CONTENTS.yaml``; ``arguments <shortname>...``
prints the framework arguments that select a sample configuration and the benchmark scenarios (with their trainer
arguments) that use it.
"""
from __future__ import annotations

import argparse
import importlib
import os
import sys

import yaml

from .constants import PLUGINS

REPO_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
CONTENTS = os.path.join(REPO_ROOT, "sample-configurations", "CONTENTS.yaml")
PLUGIN_LONG_NAMES = {
    "peft": "accelerated-peft", "foak": "fused-ops-and-kernels", "aadp": "attention-and-distributed-packing",
    "moe": "accelerated-moe", "odm": "online-data-mixing", "mcp": "mamba-cp",
}


def _plugin_status(short: str) -> bool:
    try:
        importlib.import_module(f"fms_acceleration_b200.plugins.{short}")
        return True
    except Exception:
        return False


def install(plugin: str = None, build: bool = False, **kwargs) -> int:
    known = set(PLUGINS) | set(PLUGIN_LONG_NAMES.values())
    if plugin is not None and plugin.replace("fms-acceleration-", "") not in known:
        print(f"unknown plugin '{plugin}'; available: {sorted(PLUGIN_LONG_NAMES.values())}")
        return 1
    print("all plugins are part of this package; nothing to download")
    if build:
        from ..build import build as _build

        print("native library:", _build())
    return 0


def install_plugin(*args: str) -> int:
    """Name and calling convention of the reference's verb (fms_acceleration/cli.py:36-96): one plugin name plus
    optional pip-style flags.  Every plugin ships inside this package, so the flags are accepted and ignored and
    nothing is downloaded; an unknown name is an error."""
    names = [a for a in args if not a.startswith("-")]
    if len(names) != 1:
        raise ValueError("Please specify exactly one plugin to install")
    name = os.path.basename(names[0].format(toxinidir=os.getcwd()).rstrip("/"))
    return install(name.replace("fms_acceleration_", "").replace("fms-acceleration-", ""))


def get_benchmark_artifacts(dest_dir: str) -> str:
    """Place the benchmark harness and the sample configurations under ``dest_dir`` (the reference sparse-checks them
    out of its repository, fms_acceleration/cli.py:99-120; here they are copied from this installation)."""
    import shutil

    os.makedirs(dest_dir, exist_ok=True)
    bench_src = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "benchmarks")
    pairs = [(bench_src, os.path.join(dest_dir, "scripts", "benchmarks")),
             (os.path.dirname(CONTENTS), os.path.join(dest_dir, "sample-configurations"))]
    for src, dst in pairs:
        if not os.path.isdir(src):
            raise RuntimeError(f"could not get benchmark artifacts: {src} is not part of this installation")
        shutil.copytree(src, dst, dirs_exist_ok=True, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
    return dest_dir


def list_plugins() -> int:
    print("\nplugins (x = importable):\n")
    for short in PLUGINS:
        mark = "x" if _plugin_status(short) else " "
        print(f" [{mark}] {short:5s} {PLUGIN_LONG_NAMES[short]}")
    return 0


def _read_contents():
    with open(CONTENTS, encoding="utf-8") as fh:
        return yaml.safe_load(fh)["framework_configs"]


def list_sample_configs() -> int:
    print(f"\nsample configurations ({os.path.dirname(CONTENTS)}):\n")
    for i, c in enumerate(_read_contents(), 1):
        print(f"{i:2d}. {c['shortname']:48s} plugins: {', '.join(c['plugins'])}")
    return 0


def list_arguments(*config_shortnames: str, scenario_file: str = None, ignored_fields=None) -> int:
    """For every sample configuration named: the framework arguments that select it, then (as the reference's verb
    prints, fms_acceleration/cli.py:139-186) the benchmark scenarios that use it with their trainer arguments."""
    ignored_fields = ["model_name_or_path"] if ignored_fields is None else ignored_fields
    contents = {c["shortname"]: c for c in _read_contents()}
    unknown = [n for n in config_shortnames if n not in contents]
    for name in unknown:
        print(f"no sample configuration with shortname '{name}'; see the `configs` verb")
    for name in config_shortnames:
        if name in contents:
            c = contents[name]
            path = os.path.join(os.path.dirname(CONTENTS), c["filename"])
            print(f"--acceleration_framework_config_file {path}")
            print(f"(or: export ACCELERATION_FRAMEWORK_CONFIG_FILE={path})")
            print("required plugins: " + ", ".join(c["plugins"]))
    scenario_file = scenario_file or os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))),
                                                  "benchmarks", "scenarios.yaml")
    found = 0
    if os.path.isfile(scenario_file):
        with open(scenario_file, encoding="utf-8") as fh:
            scenarios = yaml.safe_load(fh)["scenarios"]
        for scn in scenarios:
            hits = [n for n in config_shortnames if n in (scn.get("framework_config") or [])]
            if not hits:
                continue
            found += 1
            print(f"{found}. scenario: {scn['name']}\n   configs: {', '.join(hits)}\n   arguments:")
            lines = [f"      --{k} {v}" for k, v in (scn.get("arguments") or {}).items() if k not in ignored_fields]
            print(" \\\n".join(lines) + "\n")
    return 1 if unknown else 0


def cli(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="fms_acceleration.cli")
    sub = ap.add_subparsers(dest="verb", required=True)
    p = sub.add_parser("install", help="install a plugin (all plugins ship with this package)")
    p.add_argument("plugin", nargs="?")
    p.add_argument("--build", action="store_true", help="(re)build the native CUDA/C++ library")
    sub.add_parser("plugins", help="list plugins")
    sub.add_parser("configs", help="list sample configurations")
    p = sub.add_parser("arguments", help="print the arguments for one or more sample configurations")
    p.add_argument("config_shortname", nargs="+")
    a, extra = ap.parse_known_args(argv)
    if a.verb == "install":
        # pip-style flags of the reference's verb (-e, --no-deps, ...) have nothing to act on here
        flags = [x for x in extra if x.startswith("-")]
        names = [x for x in extra if not x.startswith("-")]
        if a.plugin is None and len(names) == 1:
            a.plugin = os.path.basename(names.pop().rstrip("/"))
        if names:
            ap.error("Please specify exactly one plugin to install")
        if flags:
            print(f"ignored installer flags: {' '.join(flags)}")
        plugin = a.plugin
        if plugin is not None:
            plugin = os.path.basename(plugin.rstrip("/")).replace("fms_acceleration_", "").replace("fms-acceleration-", "")
        return install(plugin, a.build)
    if extra:
        ap.error(f"unrecognized arguments: {' '.join(extra)}")
    if a.verb == "plugins":
        return list_plugins()
    if a.verb == "configs":
        return list_sample_configs()
    return list_arguments(*a.config_shortname)


if __name__ == "__main__":
    sys.exit(cli())
