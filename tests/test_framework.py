"""Framework core: configuration matching (AND / OR key paths), plugin activation rules, lifecycle dispatch."""
import pytest
import torch
import yaml

from fms_acceleration_b200.framework import (AccelerationFramework, AccelerationPlugin, AccelerationPluginConfigError,
                                             get_relevant_configuration_sections)
from fms_acceleration_b200.framework.constants import ACCELERATION_FRAMEWORK_ENV_KEY, KEY_PLUGINS
from fms_acceleration_b200.framework.utils.test_utils import (build_framework_and_maybe_instantiate,
                                                              configure_framework_from_json,
                                                              create_noop_model_with_archs, create_plugin_cls,
                                                              dummy_augmentation, dummy_custom_loader,
                                                              update_configuration_contents)


def test_config_with_empty_body_raises(tmp_path):
    p = tmp_path / "c.yaml"
    p.write_text(yaml.dump({KEY_PLUGINS: None}))
    with pytest.raises(ValueError, match="Configuration file must contain"):
        AccelerationFramework(str(p))


def test_no_config_and_no_env_raises(monkeypatch):
    monkeypatch.delenv(ACCELERATION_FRAMEWORK_ENV_KEY, raising=False)
    with pytest.raises(ValueError, match="is not set"):
        AccelerationFramework()


def test_and_or_configuration_matching():
    A = create_plugin_cls("A")
    B = create_plugin_cls("B")
    C = create_plugin_cls("C")
    cfg = {"x": {"y": {"k": 1}}, "z": {"w": 2}, "o": {"p": 3}}
    with build_framework_and_maybe_instantiate(
        [(["x.y", "z"], A), (["x.y", "missing"], B), ([], ["nope", "o.p"], C)], instantiate=False
    ):
        got = get_relevant_configuration_sections(cfg)
    names = [cls.__name__ for _, cls in got]
    assert names == ["A", "C"]
    sec_a = dict(got)[0] if False else got[0][0]
    assert sec_a == {"x": {"y": {"k": 1}}, "z": {"w": 2}}
    assert got[1][0] == {"o": {"p": 3}}


def test_or_path_rescues_missing_and_path():
    A = create_plugin_cls("A")
    with build_framework_and_maybe_instantiate([(["gone"], ["here"], A)], instantiate=False):
        got = get_relevant_configuration_sections({"here": {"v": 1}})
    assert [c.__name__ for _, c in got] == ["A"] and got[0][0] == {"here": {"v": 1}}


def test_no_plugin_matches_raises():
    A = create_plugin_cls("A")
    with pytest.raises(ValueError, match="No plugins could be configured"):
        with build_framework_and_maybe_instantiate([(["a.b"], A)], {"other": {"key": 1}}):
            pass


def test_single_plugin_lifecycle_and_arch_restriction():
    model_ok = create_noop_model_with_archs(archs=["CanDo"])()
    model_bad = create_noop_model_with_archs(archs=["CannotDo"])()
    P = create_plugin_cls("P", restricted_models={"CanDo"}, requires_augmentation=True, augmentation=dummy_augmentation)
    with build_framework_and_maybe_instantiate([(["dummy"], P)], {"dummy": {"key1": 1}}) as fw:
        assert fw.requires_augmentation and not fw.requires_custom_loading
        m, args = fw.augmentation(model_ok, None, modifiable_args=("x",))
        assert m is model_ok and args == ("x",)
        with pytest.raises(ValueError, match="are not supported for"):
            fw.augmentation(model_bad, None, modifiable_args=())
        with pytest.raises(NotImplementedError, match="require custom loading"):
            fw.model_loader("anything")


def test_at_most_one_loader_plugin():
    L1 = create_plugin_cls("L1", requires_custom_loading=True, model_loader=dummy_custom_loader)
    L2 = create_plugin_cls("L2", requires_custom_loading=True, model_loader=dummy_custom_loader)
    with pytest.raises(AssertionError, match="at most 1 plugin with custom model loading"):
        with build_framework_and_maybe_instantiate([(["a"], L1), (["b"], L2)], {"a": {"k": 1}, "b": {"k": 1}}):
            pass
    with build_framework_and_maybe_instantiate([(["a"], L1)], {"a": {"k": 1}}) as fw:
        assert fw.requires_custom_loading
        assert fw.model_loader("x").config.architectures == ["DummyModel"]


def test_activation_order_follows_registration_order():
    order = []

    def aug(tag):
        def _a(self, model, train_args, modifiable_args):
            order.append(tag)
            return model, modifiable_args
        return _a

    plugins = [create_plugin_cls(f"P{i}", requires_augmentation=True, augmentation=aug(i)) for i in range(3)]
    cfg = {f"k{i}": {"v": i} for i in range(3)}
    with build_framework_and_maybe_instantiate([([f"k{i}"], p) for i, p in enumerate(plugins)], cfg) as fw:
        fw.augmentation(create_noop_model_with_archs()(), None, modifiable_args=())
    assert order == [0, 1, 2]
    order.clear()
    with build_framework_and_maybe_instantiate([([f"k{i}"], plugins[i]) for i in (2, 0, 1)], cfg) as fw:
        fw.augmentation(create_noop_model_with_archs()(), None, modifiable_args=())
    assert order == [2, 0, 1]


def test_missing_required_package():
    P = create_plugin_cls("P", require_pkgs={"surely_not_installed_pkg"})
    with pytest.raises(ValueError, match="required by activated plugin 'P'"):
        with build_framework_and_maybe_instantiate([(["a"], P)], {"a": {"k": 1}}):
            pass
    with build_framework_and_maybe_instantiate([(["a"], P)], {"a": {"k": 1}}, require_packages_check=False) as fw:
        assert [n for n, _ in fw.active_plugins] == ["P"]


def test_env_variable_config(tmp_path, monkeypatch):
    P = create_plugin_cls("P")
    f = tmp_path / "c.yaml"
    f.write_text(yaml.dump({KEY_PLUGINS: {"a": {"k": 1}}}))
    monkeypatch.setenv(ACCELERATION_FRAMEWORK_ENV_KEY, str(f))
    with build_framework_and_maybe_instantiate([(["a"], P)], instantiate=False):
        fw = AccelerationFramework()
        assert [n for n, _ in fw.active_plugins] == ["P"]


def test_config_value_validators():
    class V(AccelerationPlugin):
        def __init__(self, cfg):
            super().__init__(cfg)
            self.kind = self._check_config_and_maybe_check_values("sec.kind", ["a", "b"])
            self.opt = self._check_config_and_maybe_check_values("sec.opt", [1, 2], default=2)
            self._check_config_equal("sec.fixed", True)

    assert V({"sec": {"kind": "a", "fixed": True}}).opt == 2
    with pytest.raises(AccelerationPluginConfigError, match="Not found in expected set"):
        V({"sec": {"kind": "c", "fixed": True}})
    with pytest.raises(AccelerationPluginConfigError):
        V({"sec": {"kind": "a", "fixed": False}})
    with pytest.raises(AccelerationPluginConfigError, match="was not a valid configuration"):
        V({"sec": {"kind": "a", "fixed": True}})._check_config_and_maybe_check_values("sec.absent")


def test_update_configuration_contents_renames_dict_keys():
    cfg = {"a": {"b": {"c": 1}}, "d": 2}
    update_configuration_contents(cfg, "a.b", "renamed")
    assert cfg == {"a": {"renamed": {"c": 1}}, "d": 2}
    update_configuration_contents(cfg, "d", 5)
    assert cfg["d"] == 5


def test_callbacks_collected_and_patchers_run():
    from fms_acceleration_b200.compat import Accelerator
    from fms_acceleration_b200.framework.utils.test_utils import instantiate_accel_patcher, instantiate_model_patcher

    class CB(AccelerationPlugin):
        def get_callbacks_and_ready_for_train(self, model=None, accelerator=None):
            return ["cb-from-plugin"]

    with instantiate_model_patcher(), instantiate_accel_patcher():
        with build_framework_and_maybe_instantiate([(["a"], CB)], {"a": {"k": 1}}) as fw:
            cbs = fw.get_callbacks_and_ready_for_train(torch.nn.Linear(2, 2), Accelerator(device="cpu"))
    assert cbs == ["cb-from-plugin"]


def test_configure_framework_from_json_builds_from_a_dict():
    """The helper writes ``{plugins: contents}`` to a temporary YAML file and builds the framework from it."""
    P = create_plugin_cls("FromJson", requires_augmentation=True, augmentation=dummy_augmentation)
    with build_framework_and_maybe_instantiate([(["json_section"], P)], instantiate=False):
        fw = configure_framework_from_json({"json_section": {"k": 1}}, require_packages_check=False)
        assert [name for name, _ in fw.active_plugins] == ["FromJson"]
        AccelerationFramework.reset()  # the active-plugin lists are class attributes, as in the reference
        with pytest.raises(ValueError, match="No plugins could be configured"):
            configure_framework_from_json({"other_section": {"k": 1}}, require_packages_check=False)
