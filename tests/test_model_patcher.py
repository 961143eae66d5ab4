"""ModelPatcher / AcceleratorPatcher rule engines."""
import importlib
import sys
import textwrap
import warnings

import pytest
import torch
from torch.utils.data import DataLoader

from fms_acceleration_b200.framework.accelerator_patcher import AcceleratorPatcher, AcceleratorPatcherComponent
from fms_acceleration_b200.framework.model_patcher import (ModelPatcher, ModelPatcherRule, ModelPatcherTrigger,
                                                           ModelPatcherTriggerType, combine_functions,
                                                           combine_triggers, patch_target_module)
from fms_acceleration_b200.framework.utils.test_utils import instantiate_accel_patcher, instantiate_model_patcher


class Leaf(torch.nn.Module):
    def forward(self, x):
        return x + 1


class Other(torch.nn.Module):
    def forward(self, x):
        return x * 10


class Tree(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.a = Leaf()
        self.b = Leaf()
        self.c = Other()

    def forward(self, x):
        return self.c(self.b(self.a(x)))


def test_trigger_construction_and_types():
    t = ModelPatcherTrigger(check=Leaf)
    assert t.type == ModelPatcherTriggerType.module and t.is_triggered(Leaf()) and not t.is_triggered(Other())
    t2 = ModelPatcherTrigger(check=lambda m: isinstance(m, Other))
    assert t2.type == ModelPatcherTriggerType.callable and t2.is_triggered(Other())
    with pytest.raises(TypeError):
        ModelPatcherTrigger(check=5)
    with pytest.raises(AssertionError):
        ModelPatcherTrigger(check=Leaf, type=ModelPatcherTriggerType.callable)
    named = ModelPatcherTrigger(check=Leaf, module_name="a")
    assert named.is_triggered(Leaf(), "a") and not named.is_triggered(Leaf(), "b")
    # a predicate that throws simply does not fire
    assert not ModelPatcherTrigger(check=lambda m: m.nope).is_triggered(Leaf())


def test_combine_triggers_and_functions():
    ta, tb = ModelPatcherTrigger(check=Leaf), ModelPatcherTrigger(check=lambda m: hasattr(m, "flag"))
    m = Leaf()
    assert combine_triggers(ta, tb, logic="OR").is_triggered(m)
    assert not combine_triggers(ta, tb, logic="AND").is_triggered(m)
    m.flag = True
    assert combine_triggers(ta, tb, logic="AND").is_triggered(m)
    with pytest.raises(AssertionError):
        combine_triggers(ta, tb, logic="XOR")
    f = combine_functions(lambda x: [x], lambda x: [x + 1, x + 2])
    assert f(1) == [1, 2, 3]


def test_rule_validation():
    with pytest.raises(ValueError, match="at most one"):
        ModelPatcherRule("r", forward=lambda s, x: x, forward_builder=lambda m: None)
    with pytest.raises(ValueError, match="trigger must be None"):
        ModelPatcherRule("r", trigger=ModelPatcherTrigger(check=Leaf), import_and_maybe_reload=("a.b", 1, None))
    with pytest.raises(ValueError, match="no forward_builder"):
        ModelPatcherRule("r", forward_builder_args=["x"])


def test_forward_rule_first_match_wins_and_history():
    with instantiate_model_patcher():
        ModelPatcher.register(ModelPatcherRule("leaf-x2", trigger=ModelPatcherTrigger(check=Leaf),
                                               forward=lambda self, x: x * 2))
        ModelPatcher.register(ModelPatcherRule("leaf-x3", trigger=ModelPatcherTrigger(check=Leaf),
                                               forward=lambda self, x: x * 3))
        with pytest.raises(AssertionError, match="already exists"):
            ModelPatcher.register(ModelPatcherRule("leaf-x2"))
        model = Tree()
        with warnings.catch_warnings(record=True) as w:
            warnings.simplefilter("always")
            ModelPatcher.patch(model)
        assert any("is ignored" in str(x.message) for x in w)
        assert model(torch.tensor(1.0)).item() == 40.0  # (1*2*2)*10
        assert sorted(h.module_name for h in ModelPatcher.history) == ["a", "b"]
        s = ModelPatcher.summary()
        assert "leaf-x2" in s and "Num:  1" in s
        assert len(ModelPatcher.summary(raw=True)) == 2


def test_forward_builder_with_nested_isolated_patch():
    with instantiate_model_patcher():
        def builder(mod):
            return [(ModelPatcherTrigger(check=Leaf, module_name="a"), lambda self, x: x + 100),
                    (ModelPatcherTrigger(check=Other), lambda self, x: x * 0)]

        ModelPatcher.register(ModelPatcherRule("tree", trigger=ModelPatcherTrigger(check=Tree), forward_builder=builder))
        model = Tree()
        ModelPatcher.patch(model)
        # a -> +100, b untouched (+1), c -> *0
        assert model.a(torch.tensor(0.0)).item() == 100 and model.b(torch.tensor(0.0)).item() == 1
        assert model(torch.tensor(1.0)).item() == 0
        ids = sorted(h.rule_id for h in ModelPatcher.history)
        assert ids == ["tree-1", "tree-2"]
        assert set(ModelPatcher.rules) == {"tree"}  # the temporary nested rules are gone


def test_forward_builder_receives_selected_kwargs():
    with instantiate_model_patcher():
        seen = {}

        def builder(mod, scale=None):
            seen["scale"] = scale
            return lambda self, x: x * scale

        ModelPatcher.register(ModelPatcherRule("b", trigger=ModelPatcherTrigger(check=Other), forward_builder=builder,
                                               forward_builder_args=["scale"]))
        m = Tree()
        ModelPatcher.patch(m, scale=7, unrelated=1)
        assert seen == {"scale": 7} and m.c(torch.tensor(1.0)).item() == 7


def _write_pkg(tmp_path, name, files):
    root = tmp_path / name
    root.mkdir()
    for fn, src in files.items():
        (root / fn).write_text(textwrap.dedent(src))
    sys.path.insert(0, str(tmp_path))
    importlib.invalidate_caches()


def test_import_and_reload_rules(tmp_path):
    _write_pkg(tmp_path, "mp_fix", {
        "__init__.py": "",
        "lib.py": "def helper():\n    return 'orig'\n",
        "user.py": """
            import torch
            from mp_fix.lib import helper
            class M(torch.nn.Module):
                def forward(self, x):
                    return helper()
        """,
    })
    try:
        import mp_fix.user as user

        with instantiate_model_patcher():
            ModelPatcher.register(ModelPatcherRule(
                "reload", import_and_maybe_reload=("mp_fix.lib.helper", lambda: "patched", "mp_fix.user")))
            m = user.M()
            ModelPatcher.patch(m)
            # the consumer module was reloaded while the replacement was in place ...
            assert sys.modules["mp_fix.user"].helper() == "patched"
            # ... and the source module has its original object back
            assert sys.modules["mp_fix.lib"].helper() == "orig"
            assert [h.rule_id for h in ModelPatcher.history] == ["reload"]

        # permanent replacement (no reload target)
        patch_target_module("mp_fix.lib.helper", lambda: "perm")
        assert sys.modules["mp_fix.lib"].helper() == "perm"
    finally:
        sys.path.remove(str(tmp_path))
        for k in [k for k in sys.modules if k.startswith("mp_fix")]:
            del sys.modules[k]


def test_conflicting_reload_targets_rejected(tmp_path):
    _write_pkg(tmp_path, "mp_fix2", {"__init__.py": "", "lib.py": "A = 1\nB = 2\n", "sub.py": "import torch\nclass M(torch.nn.Module):\n    pass\n"})
    try:
        import mp_fix2.sub as sub

        with instantiate_model_patcher():
            ModelPatcher.register(ModelPatcherRule("r1", import_and_maybe_reload=("mp_fix2.lib.A", 10, "mp_fix2")))
            ModelPatcher.register(ModelPatcherRule("r2", import_and_maybe_reload=("mp_fix2.lib.B", 20, "mp_fix2.sub")))
            m = sub.M()
            m.__class__.__module__ = "mp_fix2"
            with pytest.raises(AssertionError, match="multiple times"):
                ModelPatcher.patch(m)
    finally:
        sys.path.remove(str(tmp_path))
        for k in [k for k in sys.modules if k.startswith("mp_fix2")]:
            del sys.modules[k]


# ---------------------------------------------------------------------------------------------- accelerator
class _Acc:
    def __init__(self):
        self.prepared = []
        self.is_main_process = True

    def prepare(self, *args, device_placement=None):
        self.prepared.append(args)
        return args[0] if len(args) == 1 else args


def test_accelerator_patcher_rule_validation():
    with instantiate_accel_patcher():
        with pytest.raises(AssertionError, match="either replacement or replacement_builder"):
            AcceleratorPatcher.replace("r", AcceleratorPatcherComponent.data_collator)
        with pytest.raises(AssertionError, match="wrong type"):
            AcceleratorPatcher.replace("r", AcceleratorPatcherComponent.data_loader, replacement=5)
        with pytest.raises(AssertionError, match="Invalid special behavior"):
            AcceleratorPatcher.replace("r", AcceleratorPatcherComponent.data_collator, replacement=lambda x: x, bogus=1)
        AcceleratorPatcher.replace("ok", AcceleratorPatcherComponent.data_collator, replacement=lambda x: x)
        with pytest.raises(AssertionError, match="already been called once"):
            AcceleratorPatcher.replace("again", AcceleratorPatcherComponent.data_collator, replacement=lambda x: x)


def test_collator_replacement_and_prereq():
    ds = [{"v": i} for i in range(4)]
    with instantiate_accel_patcher():
        AcceleratorPatcher.replace("coll", AcceleratorPatcherComponent.data_collator,
                                   replacement_builder=lambda old: (lambda feats: "NEW"),
                                   pre_requisite_check=lambda c: getattr(c, "tag", None) == "good")
        acc = _Acc()
        AcceleratorPatcher.patch(acc)

        def good(f):
            return f
        good.tag = "good"
        dl = acc.prepare(DataLoader(ds, batch_size=2, collate_fn=good))
        assert next(iter(dl)) == "NEW" and len(acc.prepared) == 1
        with pytest.raises(AssertionError, match="failed pre-requisite check"):
            acc.prepare(DataLoader(ds, batch_size=2, collate_fn=lambda f: f))
        # non-dataloader arguments pass straight through
        assert acc.prepare("model", "opt") == ("model", "opt")
        assert "coll" in AcceleratorPatcher.summary()


def test_dataloader_replacement_with_skip_prepare():
    ds = list(range(6))
    replacement = DataLoader(ds, batch_size=3)
    with instantiate_accel_patcher():
        AcceleratorPatcher.replace("dl", AcceleratorPatcherComponent.data_loader, replacement=replacement, skip_prepare=True)
        acc = _Acc()
        AcceleratorPatcher.patch(acc)
        out = acc.prepare(DataLoader(ds, batch_size=1))
        assert out is replacement and acc.prepared == []
