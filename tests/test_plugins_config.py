"""Every plugin is activated by its own configuration file and rejects wrong key paths / values."""
import copy
import os

import pytest
import yaml

import fms_acceleration_b200.plugins  # noqa: F401  (registers the plugins)
from fms_acceleration_b200.framework import AccelerationPluginConfigError
from fms_acceleration_b200.framework.generate_sample_configurations import COMBINATIONS, generate
from fms_acceleration_b200.framework.utils.test_utils import (instantiate_framework, read_configuration,
                                                              update_configuration_contents)

CFG_DIR = os.path.join(os.path.dirname(fms_acceleration_b200.plugins.__file__))


def _cfg(rel):
    return read_configuration(os.path.join(CFG_DIR, rel))


@pytest.mark.parametrize("rel,expected", [
    ("peft/configs/bnb.yaml", ["BNBAccelerationPlugin"]),
    ("peft/configs/autogptq.yaml", ["AutoGPTQAccelerationPlugin"]),
    ("foak/configs/fast_kernels.yaml", ["FastKernelsAccelerationPlugin"]),
    ("foak/configs/fast_quantized_peft.yaml", ["FastKernelsAccelerationPlugin"]),
    ("aadp/configs/padding_free.yaml", ["PaddingFreeAccelerationPlugin"]),
])
def test_plugin_activated_by_its_config(rel, expected):
    with instantiate_framework(_cfg(rel), require_packages_check=False) as fw:
        assert [n for n, _ in fw.active_plugins] == expected


def test_bnb_plugin_flags_and_values():
    cfg = _cfg("peft/configs/bnb.yaml")
    with instantiate_framework(cfg) as fw:
        assert fw.requires_custom_loading and fw.requires_augmentation
    baseline = update_configuration_contents(copy.deepcopy(cfg), "peft.quantization.bitsandbytes.no_peft_model", True)
    with instantiate_framework(baseline) as fw:
        assert fw.requires_custom_loading and not fw.requires_augmentation
    bad = update_configuration_contents(copy.deepcopy(cfg), "peft.quantization.bitsandbytes.quant_type", "int3")
    with pytest.raises(AccelerationPluginConfigError, match="quant_type"):
        with instantiate_framework(bad):
            pass


def test_wrong_key_path_configures_nothing():
    cfg = _cfg("peft/configs/bnb.yaml")
    renamed = update_configuration_contents(copy.deepcopy(cfg), "peft.quantization.bitsandbytes", "something_else")
    with pytest.raises(ValueError, match="No plugins could be configured"):
        with instantiate_framework(renamed):
            pass


def test_autogptq_rejects_other_kernels():
    cfg = _cfg("peft/configs/autogptq.yaml")
    for key, val in (("peft.quantization.auto_gptq.kernel", "cuda"), ("peft.quantization.auto_gptq.from_quantized", False)):
        bad = update_configuration_contents(copy.deepcopy(cfg), key, val)
        with pytest.raises(AccelerationPluginConfigError):
            with instantiate_framework(bad):
                pass


def test_two_loader_plugins_conflict():
    cfg = _cfg("peft/configs/bnb.yaml")
    cfg["peft"]["quantization"].update(_cfg("peft/configs/autogptq.yaml")["peft"]["quantization"])
    with pytest.raises(AssertionError, match="at most 1 plugin"):
        with instantiate_framework(cfg):
            pass


def test_foak_options_and_filter_terms():
    cfg = _cfg("foak/configs/fast_quantized_peft.yaml")
    with instantiate_framework(cfg) as fw:
        plugin = dict(fw.active_plugins)["FastKernelsAccelerationPlugin"]
        assert plugin.configurations["base_layer"] == "auto_gptq"
        assert plugin.selected_terms(quantised=True) == {"qkvo", "mlp", "cross-ent", "custom-loss", "rms", "rope"}
        assert plugin.selected_terms(quantised=False) == {"cross-ent", "custom-loss", "rms", "rope"}
    liger = _cfg("foak/configs/fast_quantized_peft_liger.yaml")
    with instantiate_framework(liger) as fw:
        plugin = dict(fw.active_plugins)["FastKernelsAccelerationPlugin"]
        # the sample file spells the norm key differently, so the real option keeps its default
        assert plugin.configurations["fast_rms_layernorm"] is False
        assert plugin.selected_terms(quantised=True) == {"qkvo", "mlp", "fused-lce", "rope"}
    bad = update_configuration_contents(copy.deepcopy(cfg), "peft.quantization.fused_ops_and_kernels.fast_loss", "maybe")
    with pytest.raises(AccelerationPluginConfigError):
        with instantiate_framework(bad):
            pass


def test_multipack_needs_padding_free_section():
    mp = _cfg("aadp/configs/multipack.yaml")
    with pytest.raises(ValueError, match="No plugins could be configured"):
        with instantiate_framework(mp):
            pass
    both = copy.deepcopy(mp)
    both["training"].update(_cfg("aadp/configs/padding_free.yaml")["training"])
    with instantiate_framework(both) as fw:
        assert [n for n, _ in fw.active_plugins] == ["PaddingFreeAccelerationPlugin", "MultipackDataloaderAccelerationPlugin"]


def test_sample_configurations_are_current_and_loadable():
    files = generate()
    assert len(files) == 27 and len(COMBINATIONS) == 26
    out_dir = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "sample-configurations")
    for name, text in files.items():
        with open(os.path.join(out_dir, name), encoding="utf-8") as fh:
            assert fh.read() == text, f"{name} is stale: re-run the generator"
    contents = yaml.safe_load(files["CONTENTS.yaml"])["framework_configs"]
    assert {c["shortname"] for c in contents} >= {"accelerated-peft-bnb-foak", "aadp-padding-free-multipack",
                                                  "moe-scattermoe-granite-ep8-foak"}
    for c in contents:
        body = yaml.safe_load(files[c["filename"]])
        assert "plugins" in body and body["plugins"]


def test_rule_filter_keeps_or_drops_by_id_suffix():
    """Rule-id suffix filtering of the fused-ops plugin (intent of the reference's tests/test_model_utils.py)."""
    from fms_acceleration_b200.framework.model_patcher import ModelPatcherRule
    from fms_acceleration_b200.plugins.foak.utils import filter_mp_rules

    fwd = lambda self, x: x  # noqa: E731
    ids = ["llama-rms", "llama-qkvo", "llama-mlp", "llama-rope", "llama-fused-lce", "llama-custom-loss"]
    rules = [ModelPatcherRule(rule_id=i, forward=fwd) for i in ids]
    kept = filter_mp_rules(rules, {"qkvo", "mlp"})
    assert [r.rule_id for r in kept] == ["llama-qkvo", "llama-mlp"]
    dropped = filter_mp_rules(rules, {"qkvo", "mlp"}, drop=True)
    assert [r.rule_id for r in dropped] == ["llama-rms", "llama-rope", "llama-fused-lce", "llama-custom-loss"]
    assert filter_mp_rules(rules, {"nothing"}) == []
