"""Rule engine that swaps module forwards and module-level objects of a model in place.

Contract of fms_acceleration/model_patcher.py:31-574 in the reference:

* a rule has a unique ``rule_id``, an optional ``trigger`` and at most one of ``forward`` (bound as the
  module's new ``forward``), ``forward_builder`` (called with the module, returns a forward or a list of
  ``(trigger, forward)`` pairs that are applied as an isolated nested patch of that module's children) or
  ``import_and_maybe_reload = (target_path, replacement, module_to_reload)``;
* ``ModelPatcher.patch(model)`` first performs the import/reload rules that concern the model's python
  module (rules with a reload target go first; two rules may share one reload target, but one reload
  target may not be a prefix of another), then walks ``named_modules()``: the first rule (in registration
  order) whose trigger fires wins, later plain-forward matches on the same module only warn;
* every application is recorded in ``ModelPatcher.history`` and summarised by ``ModelPatcher.summary()``.

One deliberate difference: the name a trigger sees is always the last component of the module's dotted
name (the reference passes the first component for names of up to two parts,
model_patcher.py:407-419, which makes name triggers unreliable outside nested patches).
"""
from __future__ import annotations

import importlib
import importlib.util
import inspect
import warnings
from collections import OrderedDict
from dataclasses import asdict, dataclass
from enum import Enum
from types import MethodType
from typing import Any, Callable, Dict, List, Optional, Set, Tuple, Type, Union

import torch


def patch_target_module(to_patch: str, replace_with: Any, target_module: Optional[str] = None) -> None:
    """Replace the object at dotted path ``to_patch``.

    Without ``target_module`` the replacement is permanent.  With it, the replacement is only in effect
    while ``target_module`` is re-imported (so that its ``from x import y`` statements bind the
    replacement) and the original object is restored afterwards.
    """
    parts = to_patch.split(".")
    assert len(parts) > 1, "must have an object to patch"
    owner = importlib.import_module(".".join(parts[:-1]))
    attr = parts[-1]
    original = getattr(owner, attr)
    setattr(owner, attr, replace_with)
    if target_module is not None:
        try:
            importlib.reload(importlib.import_module(target_module))
        finally:
            setattr(owner, attr, original)


class ModelPatcherTriggerType(Enum):
    module = 1
    callable = 2


@dataclass
class ModelPatcherTrigger:
    """Decides whether a rule applies to a module: an ``nn.Module`` subclass (isinstance test) or a
    predicate ``module -> bool``; optionally also restricted to a module name."""

    check: Union[Type[torch.nn.Module], Callable[[torch.nn.Module], bool]]
    type: Optional[ModelPatcherTriggerType] = None
    module_name: Optional[str] = None

    def __post_init__(self):
        if inspect.isclass(self.check) and issubclass(self.check, torch.nn.Module):
            inferred = ModelPatcherTriggerType.module
        elif callable(self.check):
            inferred = ModelPatcherTriggerType.callable
        else:
            raise TypeError("check argument needs to be torch.nn.Module or Callable")
        if self.type is None:
            self.type = inferred
        else:
            assert self.type == inferred, "type argument passed but `check` argument does not match type specified"

    def is_triggered(self, module: torch.nn.Module, module_name: Optional[str] = None) -> bool:
        if self.module_name is not None and module_name != self.module_name:
            return False
        if self.type == ModelPatcherTriggerType.module:
            return isinstance(module, self.check)
        try:
            return bool(self.check(module))
        except Exception:  # a predicate that cannot evaluate a module simply does not fire
            return False


ModelForward = Callable


@dataclass
class ModelPatcherRule:
    rule_id: str
    trigger: Optional[ModelPatcherTrigger] = None
    forward: Optional[ModelForward] = None
    forward_builder: Optional[Callable] = None
    forward_builder_args: Optional[List[str]] = None
    import_and_maybe_reload: Optional[Tuple[str, Any, Optional[str]]] = None

    def __post_init__(self):
        chosen = [self.forward is not None, self.forward_builder is not None, self.import_and_maybe_reload is not None]
        if sum(chosen) > 1:
            raise ValueError(
                f"Rule '{self.rule_id}' must only have at most one of forward, "
                "forward builder, or import_and_maybe_reload, specified."
            )
        if self.import_and_maybe_reload is not None and self.trigger is not None:
            raise ValueError(
                f"Rule '{self.rule_id}' has import_and_maybe_reload specified, and trigger must be None."
            )
        if self.forward_builder_args is not None and self.forward_builder is None:
            raise ValueError(f"Rule '{self.rule_id}' has forward_builder_args but no forward_builder.")


@dataclass
class ModelPatcherHistory:
    instance: int
    cls: str
    parent_cls: str
    module_name: str
    parent_module_name: str
    rule_id: str


class ModelPatcher:
    """Process-wide registry of rules plus the log of what was patched."""

    history: List[ModelPatcherHistory] = []
    rules: Dict[str, ModelPatcherRule] = OrderedDict()

    # ------------------------------------------------------------------ registration
    @staticmethod
    def load_patches(module_names: List[str], reload: bool = False) -> None:
        for name in module_names:
            if importlib.util.find_spec(name):
                mod = importlib.import_module(name)
                if reload:
                    try:
                        importlib.reload(mod)
                    except AssertionError:
                        pass  # rules of that module are already registered

    @staticmethod
    def register(rule: ModelPatcherRule) -> None:
        assert rule.rule_id not in ModelPatcher.rules, f"patch rule '{rule.rule_id}' already exists"
        ModelPatcher.rules[rule.rule_id] = rule

    @staticmethod
    def did_rule_trigger(module: torch.nn.Module, module_name: str):
        winner_id, winner = None, None
        for rule_id, rule in ModelPatcher.rules.items():
            if rule.trigger is None or not rule.trigger.is_triggered(module, module_name):
                continue
            if winner is None:
                winner_id, winner = rule_id, rule
            elif rule.forward is not None:
                warnings.warn(
                    f"rule {rule.rule_id} is ignored on {module_name} as an "
                    f"earlier rule {winner.rule_id} has been applied"
                )
        return winner_id, winner

    # ------------------------------------------------------------------ import / reload rules
    @staticmethod
    def _import_and_reload(model: torch.nn.Module) -> None:
        module_path = model.__module__
        reloading, plain = [], []
        for rule in ModelPatcher.rules.values():
            if rule.import_and_maybe_reload is None:
                continue
            target, _, reload_path = rule.import_and_maybe_reload
            if reload_path and reload_path.startswith(module_path):
                reloading.append(rule)
            elif target.startswith(module_path):
                plain.append(rule)

        # Reloading a module twice would undo the first replacement, and reloading a parent package
        # after a child is unpredictable: collapse equal targets into one reload, reject prefixes.
        reloading.sort(key=lambda r: len(r.import_and_maybe_reload[2]))
        for i, short in enumerate(reloading[:-1]):
            for long in reloading[i + 1:]:
                s_target, s_obj, s_path = short.import_and_maybe_reload
                l_path = long.import_and_maybe_reload[2]
                if s_path is None:
                    continue
                if s_path == l_path:
                    # the later rule's reload also rebinds this rule's replacement: make it permanent
                    # until then by dropping its own reload
                    short.import_and_maybe_reload = (s_target, s_obj, None)
                    continue
                assert not l_path.startswith(s_path), (
                    f"Attempting to reload a subpath`{s_path}` multiple times in "
                    f"{short.rule_id} and {long.rule_id}"
                )

        for rule in reloading + plain:
            target, obj, reload_path = rule.import_and_maybe_reload
            patch_target_module(target, obj, reload_path)
            ModelPatcher.history.append(
                ModelPatcherHistory(
                    instance=id(model), cls=model.__class__.__name__, parent_cls="", module_name="",
                    parent_module_name="", rule_id=rule.rule_id,
                )
            )

    # ------------------------------------------------------------------ forward rules
    @staticmethod
    def _patch_forwards(
        model: torch.nn.Module,
        patch_kwargs: Optional[Dict] = None,
        visited: Optional[Set] = None,
        parent_prefix: Optional[str] = None,
        parent_mcn: Optional[str] = None,
    ) -> None:
        patch_kwargs = patch_kwargs or {}
        visited = visited if visited is not None else set()

        for dotted, mod in model.named_modules():
            parts = dotted.split(".")
            module_name = parts[-1]
            if len(parts) > 1:
                parent_module_name = ".".join(parts[:-1])
                parent_cls = model.get_submodule(parent_module_name).__class__.__name__
                if parent_prefix:
                    parent_module_name = f"{parent_prefix}.{parent_module_name}"
            else:
                parent_module_name = parent_prefix or ""
                parent_cls = parent_mcn or ""

            rule_id, rule = ModelPatcher.did_rule_trigger(mod, module_name)
            if rule_id is None:
                continue

            if rule.forward is not None:
                forward = rule.forward
            elif rule.forward_builder is not None:
                kwargs = {}
                if rule.forward_builder_args is not None:
                    kwargs = {k: v for k, v in patch_kwargs.items() if k in rule.forward_builder_args}
                forward = rule.forward_builder(mod, **kwargs)
            else:
                forward = None  # trigger-only rule: record it, change nothing

            if isinstance(forward, list):
                # nested, isolated patch of this module's subtree with a temporary rule set
                saved = ModelPatcher.rules
                ModelPatcher.rules = OrderedDict()
                try:
                    for i, (trig, fwd) in enumerate(forward):
                        ModelPatcher.register(ModelPatcherRule(rule_id=f"{rule_id}-{i + 1}", trigger=trig, forward=fwd))
                    ModelPatcher._patch_forwards(
                        mod,
                        patch_kwargs=patch_kwargs,
                        visited=visited,
                        parent_prefix=(f"{parent_module_name}.{module_name}" if parent_module_name else module_name),
                        parent_mcn=mod.__class__.__name__,
                    )
                finally:
                    ModelPatcher.rules = saved
                continue

            if forward is not None:
                mod.forward = MethodType(forward, mod)
            ModelPatcher.history.append(
                ModelPatcherHistory(
                    instance=id(mod), cls=mod.__class__.__name__, parent_cls=parent_cls, module_name=module_name,
                    parent_module_name=parent_module_name, rule_id=rule_id,
                )
            )

    @staticmethod
    def patch(model: torch.nn.Module, **kwargs) -> None:
        """Apply all registered rules to ``model``.  Meant to be called once per model."""
        base = model
        getter = getattr(model, "get_base_model", None)
        if callable(getter):
            try:
                base = getter()
            except AttributeError:
                base = model
        ModelPatcher._import_and_reload(base)
        ModelPatcher._patch_forwards(model, patch_kwargs=kwargs)

    # ------------------------------------------------------------------ reporting
    @staticmethod
    def summary(raw: bool = False):
        if raw:
            import pandas as pd

            return pd.DataFrame([asdict(h) for h in ModelPatcher.history])
        if not ModelPatcher.history:
            return ""
        counts: Dict[Tuple[str, str, str], int] = {}
        for h in ModelPatcher.history:
            key = (h.rule_id, h.module_name, h.cls)
            counts[key] = counts.get(key, 0) + 1
        lines = ["***************** Module Forwards Patching *************"]
        for (rule_id, module_name, cls), num in sorted(counts.items()):
            lines.append("Rule: {0:15s} Module: {1:25s} Class: {2:15s} Num: {3:2d}".format(rule_id, module_name, cls, num))
        return "\n".join(lines)


def patch_model(model: torch.nn.Module, **kwargs) -> torch.nn.Module:
    ModelPatcher.patch(model, **kwargs)
    return model


def patch_model_summary() -> str:
    return ModelPatcher.summary()


def combine_triggers(*triggers: ModelPatcherTrigger, logic: str = "OR") -> ModelPatcherTrigger:
    assert logic in ("AND", "OR"), "Only `AND`, `OR` logic implemented for combining triggers"
    reducer = all if logic == "AND" else any

    def _combined(*args, **kwargs):
        return reducer(t.is_triggered(*args, **kwargs) for t in triggers)

    return ModelPatcherTrigger(check=_combined)


def combine_functions(*funcs: Callable, logic: str = "APPEND") -> Callable:
    assert logic == "APPEND", "only APPEND logic implemented for combining functions"

    def _appended(*args, **kwargs):
        out = []
        for f in funcs:
            out += f(*args, **kwargs)
        return out

    return _appended
