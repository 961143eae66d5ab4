"""Generate ``sample-configurations/*.yaml`` and ``CONTENTS.yaml`` from the per-plugin ``configs/*.yaml``.

Each sample configuration is the merge of one or more per-plugin configuration files, with selected keys
overridden, wrapped under the ``plugins`` root key.  File names, short names and the list of 26 combinations
are those of the reference (scripts/generate_sample_configurations.py:143-239,
sample-configurations/CONTENTS.yaml).

    python -m fms_acceleration_b200.framework.generate_sample_configurations [--out DIR] [--check]

``--check`` regenerates into memory and fails when the files on disk differ (the role of the reference's
scripts/verify_generated_configurations.sh).
"""
from __future__ import annotations

import argparse
import copy
import os
import sys
from typing import Any, Dict, List, Tuple

import yaml

from .constants import KEY_PLUGINS

PKG_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PLUGIN_CFG = os.path.join(PKG_ROOT, "plugins")
REPO_ROOT = os.path.dirname(PKG_ROOT)

# source name -> (file, [(dotted key, value)])
SOURCES: Dict[str, Tuple[str, List[Tuple[str, Any]]]] = {
    "auto-gptq": ("peft/configs/autogptq.yaml", []),
    "bnb-nf4": ("peft/configs/bnb.yaml", [("peft.quantization.bitsandbytes.quant_type", "nf4")]),
    "baseline-bnb-nf4": ("peft/configs/bnb.yaml", [("peft.quantization.bitsandbytes.quant_type", "nf4"),
                                                    ("peft.quantization.bitsandbytes.no_peft_model", True)]),
    "auto-gptq-foak": ("foak/configs/fast_quantized_peft.yaml",
                       [("peft.quantization.fused_ops_and_kernels.base_layer", "auto_gptq")]),
    "auto-gptq-foak-liger": ("foak/configs/fast_quantized_peft_liger.yaml",
                             [("peft.quantization.fused_ops_and_kernels.base_layer", "auto_gptq")]),
    "bnb-nf4-foak": ("foak/configs/fast_quantized_peft.yaml",
                     [("peft.quantization.fused_ops_and_kernels.base_layer", "bitsandbytes")]),
    "bnb-nf4-foak-liger": ("foak/configs/fast_quantized_peft_liger.yaml",
                           [("peft.quantization.fused_ops_and_kernels.base_layer", "bitsandbytes")]),
    "aadp-padding-free": ("aadp/configs/padding_free.yaml", []),
    "aadp-multipack": ("aadp/configs/multipack.yaml", []),
    "foak-fast-kernels": ("foak/configs/fast_kernels.yaml", []),
    "foak-fast-kernels-liger": ("foak/configs/fast_kernels_liger.yaml", []),
    "moe-scattermoe-ep1": ("moe/configs/scattermoe.yaml", []),
    "moe-scattermoe-ep2": ("moe/configs/scattermoe.yaml", [("training.moe.scattermoe.ep_degree", 2)]),
    "moe-scattermoe-ep4": ("moe/configs/scattermoe.yaml", [("training.moe.scattermoe.ep_degree", 4)]),
    "moe-scattermoe-ep8": ("moe/configs/scattermoe.yaml", [("training.moe.scattermoe.ep_degree", 8)]),
}

PLUGIN_OF_SOURCE = {
    "peft": "accelerated-peft", "foak": "fused-ops-and-kernels", "aadp": "attention-and-distributed-packing",
    "moe": "accelerated-moe",
}

# (file tag, short name, sources)
COMBINATIONS: List[Tuple[str, str, Tuple[str, ...]]] = [
    ("accelerated-peft-autogptq", "accelerated-peft-autogptq", ("auto-gptq",)),
    ("accelerated-peft-bnb-nf4", "accelerated-peft-bnb", ("bnb-nf4",)),
    ("baseline-peft-bnb-nf4", "baseline-peft-bnb", ("baseline-bnb-nf4",)),
    ("accelerated-peft-autogptq-foak", "accelerated-peft-autogptq-foak", ("auto-gptq", "auto-gptq-foak")),
    ("accelerated-peft-autogptq-foak-liger", "accelerated-peft-autogptq-foak-liger", ("auto-gptq", "auto-gptq-foak-liger")),
    ("accelerated-peft-bnb-nf4-foak", "accelerated-peft-bnb-foak", ("bnb-nf4", "bnb-nf4-foak")),
    ("accelerated-peft-bnb-nf4-foak-liger", "accelerated-peft-bnb-foak-liger", ("bnb-nf4", "bnb-nf4-foak-liger")),
    ("aadp-padding-free", "aadp-padding-free", ("aadp-padding-free",)),
    ("aadp-padding-free-multipack", "aadp-padding-free-multipack", ("aadp-padding-free", "aadp-multipack")),
    ("accelerated-peft-bnb-nf4-padding-free", "accelerated-peft-bnb-padding-free", ("aadp-padding-free", "bnb-nf4")),
    ("accelerated-peft-autogptq-padding-free", "accelerated-peft-autogptq-padding-free", ("aadp-padding-free", "auto-gptq")),
    ("accelerated-peft-bnb-nf4-foak-padding-free", "accelerated-peft-bnb-foak-padding-free",
     ("aadp-padding-free", "bnb-nf4", "bnb-nf4-foak")),
    ("accelerated-peft-autogptq-foak-padding-free", "accelerated-peft-autogptq-foak-padding-free",
     ("aadp-padding-free", "auto-gptq", "auto-gptq-foak")),
    ("foak-fast-kernels", "foak-fast-kernels", ("foak-fast-kernels",)),
    ("foak-fast-kernels-liger", "foak-fast-kernels-liger", ("foak-fast-kernels-liger",)),
    ("moe-scattermoe-granite-ep1", "moe-scattermoe-granite-ep1", ("moe-scattermoe-ep1",)),
    ("moe-scattermoe-granite-ep1-padding-free", "moe-scattermoe-granite-ep1-padding-free",
     ("aadp-padding-free", "moe-scattermoe-ep1")),
    ("moe-scattermoe-granite-ep1-padding-free-foak", "moe-scattermoe-granite-ep1-padding-free-foak",
     ("aadp-padding-free", "foak-fast-kernels", "moe-scattermoe-ep1")),
    ("moe-scattermoe-granite-ep2", "moe-scattermoe-granite-ep2", ("moe-scattermoe-ep2",)),
    ("moe-scattermoe-granite-ep2-padding-free", "moe-scattermoe-granite-ep2-padding-free",
     ("aadp-padding-free", "moe-scattermoe-ep2")),
    ("moe-scattermoe-granite-ep2-padding-free-foak", "moe-scattermoe-granite-ep2-padding-free-foak",
     ("aadp-padding-free", "foak-fast-kernels", "moe-scattermoe-ep2")),
    ("moe-scattermoe-granite-ep4", "moe-scattermoe-granite-ep4", ("moe-scattermoe-ep4",)),
    ("moe-scattermoe-granite-ep4-padding-free", "moe-scattermoe-granite-ep4-padding-free",
     ("aadp-padding-free", "moe-scattermoe-ep4")),
    ("moe-scattermoe-granite-ep4-padding-free-foak", "moe-scattermoe-granite-ep4-padding-free-foak",
     ("aadp-padding-free", "foak-fast-kernels", "moe-scattermoe-ep4")),
    ("moe-scattermoe-granite-ep8", "moe-scattermoe-granite-ep8", ("moe-scattermoe-ep8",)),
    ("moe-scattermoe-granite-ep8-foak", "moe-scattermoe-granite-ep8-foak", ("foak-fast-kernels", "moe-scattermoe-ep8")),
]

HEADER = "# FMS Acceleration Plugin Configuration.\n#\n# Each stanza incorporates various configurations for\n# different fine-tuning / training tasks.\n"


def _set(tree: Dict, dotted: str, value: Any) -> None:
    *parents, leaf = dotted.split(".")
    for k in parents:
        tree = tree[k]
    tree[leaf] = value


def _merge(dst: Dict, src: Dict) -> Dict:
    for k, v in src.items():
        if isinstance(v, dict) and isinstance(dst.get(k), dict):
            _merge(dst[k], v)
        else:
            dst[k] = copy.deepcopy(v)
    return dst


def load_source(name: str) -> Dict:
    rel, overrides = SOURCES[name]
    with open(os.path.join(PLUGIN_CFG, rel), encoding="utf-8") as fh:
        tree = yaml.safe_load(fh)
    for key, val in overrides:
        _set(tree, key, val)
    return tree


def render(sources: Tuple[str, ...]) -> str:
    merged: Dict = {}
    for s in sources:
        _merge(merged, load_source(s))
    return HEADER + yaml.safe_dump({KEY_PLUGINS: merged}, sort_keys=False, default_flow_style=False)


def contents_yaml() -> str:
    entries = []
    for tag, short, sources in COMBINATIONS:
        plugins = []
        for s in sources:
            p = PLUGIN_OF_SOURCE[SOURCES[s][0].split("/")[0]]
            if p not in plugins:
                plugins.append(p)
        entries.append({"shortname": short, "plugins": sorted(plugins), "filename": f"{tag}-sample-configuration.yaml"})
    head = ("# index of the sample configurations: shortname -> plugins needed -> file name\n")
    return head + yaml.safe_dump({"framework_configs": entries}, sort_keys=False, default_flow_style=False)


def generate() -> Dict[str, str]:
    files = {f"{tag}-sample-configuration.yaml": render(sources) for tag, _, sources in COMBINATIONS}
    files["CONTENTS.yaml"] = contents_yaml()
    return files


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=os.path.join(REPO_ROOT, "sample-configurations"))
    ap.add_argument("--check", action="store_true")
    ap.add_argument("output_dir", nargs="?", default=None,
                    help="where the files go: the positional form of --out, as the reference's script takes it")
    args = ap.parse_args(argv)
    if args.output_dir:
        args.out = args.output_dir
    files = generate()
    if args.check:
        bad = []
        for name, text in files.items():
            path = os.path.join(args.out, name)
            if not os.path.exists(path) or open(path, encoding="utf-8").read() != text:
                bad.append(name)
        if bad:
            print("sample configurations are out of date: " + ", ".join(bad), file=sys.stderr)
            return 1
        return 0
    os.makedirs(args.out, exist_ok=True)
    for name, text in files.items():
        with open(os.path.join(args.out, name), "w", encoding="utf-8") as fh:
            fh.write(text)
    print(f"wrote {len(files)} files to {args.out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
