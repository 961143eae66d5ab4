"""Replacement of the training data loader / data collator at ``accelerator.prepare`` time.

Contract of fms_acceleration/accelerator_patcher.py:36-279 in the reference: plugins call
``AcceleratorPatcher.replace(rule_id, component, replacement | replacement_builder, pre_requisite_check,
skip_prepare=...)`` during augmentation; ``AcceleratorPatcher.patch(accelerator)`` wraps
``accelerator.prepare`` so that a call with exactly one ``DataLoader`` argument swaps the loader and/or its
``collate_fn`` (a loader builder receives ``(dataloader, accelerator)``, a collator builder receives the old
``collate_fn``) and, with ``skip_prepare=True``, returns the new loader without the original ``prepare``.
Only one replacement per component is allowed and a failed pre-requisite check raises.

Any object with a ``prepare`` method works as the accelerator (``accelerate.Accelerator`` or the shim in
``fms_acceleration_b200.compat``).
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from types import MethodType
from typing import Any, Callable, Dict, List, Optional

from torch.utils.data import DataLoader


class AcceleratorPatcherComponent(Enum):
    data_loader = 1
    data_collator = 2


REPLACEABLE_COMPONENTS = {
    AcceleratorPatcherComponent.data_loader.value: DataLoader,
    AcceleratorPatcherComponent.data_collator.value: Callable,
}

RULE_KIND_REPLACEMENT = "replacement"
RULE_SPECIAL_KWARGS = {RULE_KIND_REPLACEMENT: {"skip_prepare"}}


@dataclass
class AcceleratorPatcherHistory:
    component: AcceleratorPatcherComponent
    kind: str
    rule_id: str


@dataclass
class AcceleratorRuleReplace:
    rule_id: str
    component: AcceleratorPatcherComponent
    replacement: Any = None
    replacement_builder: Optional[Callable] = None
    pre_req: Optional[Callable] = None
    kwargs: Optional[Dict] = None

    def __post_init__(self):
        assert (self.replacement is None) != (self.replacement_builder is None), \
            "either replacement or replacement_builder should be specified"
        self.kwargs = self.kwargs or {}
        allowed = RULE_SPECIAL_KWARGS[RULE_KIND_REPLACEMENT]
        assert all(k in allowed for k in self.kwargs), f"Invalid special behavior kwargs in '{self.kwargs.keys()}'"

    def pre_req_check(self, to_be_replaced: Any) -> None:
        if self.pre_req is None:
            return
        assert self.pre_req(to_be_replaced), (
            f"Rule '{self.rule_id}' failed pre-requisite check for type '{type(to_be_replaced)}'."
        )

    def build(self, *builder_args):
        if self.replacement is not None:
            return self.replacement
        return self.replacement_builder(*builder_args)


class AcceleratorPatcher:
    history: List[AcceleratorPatcherHistory] = []
    replacement_rules: Dict[int, AcceleratorRuleReplace] = {}

    @staticmethod
    def replace(
        rule_id: str,
        component: AcceleratorPatcherComponent,
        replacement: Any = None,
        replacement_builder: Optional[Callable] = None,
        pre_requisite_check: Optional[Callable] = None,
        **kwargs,
    ) -> None:
        """Schedule a replacement.  There is no fallback: once registered it must succeed at prepare time."""
        assert not any(h.rule_id == rule_id for h in AcceleratorPatcher.history), f"Rule '{rule_id}' has already been added"
        assert component.value not in AcceleratorPatcher.replacement_rules, (
            f"replace has already been called once on component '{component.name}'"
        )
        if replacement is not None:
            expected = REPLACEABLE_COMPONENTS.get(component.value)
            if expected is not None:
                assert isinstance(replacement, expected), (
                    f"Rule '{rule_id}' replacing component '{component}' with wrong type '{type(replacement)}'"
                )
        AcceleratorPatcher.replacement_rules[component.value] = AcceleratorRuleReplace(
            rule_id, component, replacement, replacement_builder, pre_requisite_check, kwargs=kwargs
        )
        AcceleratorPatcher.history.append(AcceleratorPatcherHistory(component, RULE_KIND_REPLACEMENT, rule_id))

    @staticmethod
    def patch(accelerator) -> None:
        wanted = {AcceleratorPatcherComponent.data_collator.value, AcceleratorPatcherComponent.data_loader.value}
        if wanted & set(AcceleratorPatcher.replacement_rules):
            AcceleratorPatcher._patch_prepare(accelerator)

    @staticmethod
    def _patch_prepare(accelerator) -> None:
        original_prepare = accelerator.prepare

        def prepare(self, *args, device_placement=None):
            if len(args) != 1 or not isinstance(args[0], DataLoader):
                return original_prepare(*args, device_placement=device_placement)

            rules = AcceleratorPatcher.replacement_rules
            loader_rule = rules.get(AcceleratorPatcherComponent.data_loader.value)
            collator_rule = rules.get(AcceleratorPatcherComponent.data_collator.value)

            dataloader = args[0]
            if loader_rule is not None:
                loader_rule.pre_req_check(dataloader)
                dataloader = loader_rule.build(dataloader, accelerator)
            if collator_rule is not None:
                collator_rule.pre_req_check(dataloader.collate_fn)
                dataloader.collate_fn = collator_rule.build(dataloader.collate_fn)
            if loader_rule is not None and loader_rule.kwargs.get("skip_prepare", False):
                return dataloader
            return original_prepare(dataloader)

        accelerator.prepare = MethodType(prepare, accelerator)

    @staticmethod
    def summary() -> str:
        lines = ["***************** Accelerator Patching *************"]
        for h in AcceleratorPatcher.history:
            lines.append("Rule: {0:25s} Kind: {1:10s} Component: {2:20s}".format(h.rule_id, h.kind, h.component.name))
        return "\n".join(lines)
