"""Helpers kept for callers that shard models themselves: re-tying of tied parameters after re-materialisation,
real storage for meta embeddings, and marking LoRA adapters as replicated."""
from types import SimpleNamespace

import torch
from torch import nn

from fms_acceleration_b200.plugins.foak.utils import lora_adapters_switch_ddp_from_fsdp
from fms_acceleration_b200.plugins.peft.fsdp_utils import ensure_weights_retied, put_selected_meta_tensors_on_cpu


class _Tied(nn.Module):
    def __init__(self, device=None):
        super().__init__()
        self.emb = nn.Embedding(8, 4, device=device)
        self.body = nn.Linear(4, 4, device=device)
        self.head = nn.Linear(4, 8, bias=False, device=device)
        self.head.weight = self.emb.weight

    def get_input_embeddings(self):
        return self.emb

    def get_output_embeddings(self):
        return self.head


def test_tied_weights_are_tied_again_after_reinitialisation():
    model = _Tied()
    calls = []

    def base_init(module):            # what a sharding engine does: give the module fresh parameters
        calls.append(type(module).__name__)
        for name, p in list(module.named_parameters(recurse=False)):
            setattr(module, name, nn.Parameter(torch.zeros_like(p)))

    init_fn = ensure_weights_retied(base_init, model, "cpu")
    for m in (model.emb, model.body, model.head):
        init_fn(m)
    assert calls == ["Embedding", "Linear", "Linear"]
    assert model.head.weight is model.emb.weight
    # nothing tied: the original function comes back untouched
    plain = nn.Sequential(nn.Linear(2, 2), nn.Linear(2, 2))
    assert ensure_weights_retied(base_init, plain, "cpu") is base_init


def test_meta_embeddings_get_cpu_storage():
    model = _Tied(device="meta")
    assert model.emb.weight.is_meta
    put_selected_meta_tensors_on_cpu(model)
    assert not model.emb.weight.is_meta and model.emb.weight.device.type == "cpu"
    assert not model.head.weight.is_meta
    assert model.body.weight.is_meta          # only the embeddings are touched


def test_adapters_are_marked_replicated_and_excluded_from_sharding():
    class _Lora(nn.Module):
        def __init__(self):
            super().__init__()
            self.base_layer = nn.Linear(4, 4)
            self.lora_A = nn.ModuleDict({"default": nn.Linear(4, 2, bias=False)})
            self.lora_B = nn.ModuleDict({"default": nn.Linear(2, 4, bias=False)})

    mods = [_Lora(), _Lora()]
    plugin = SimpleNamespace(ignored_modules=None)
    lora_adapters_switch_ddp_from_fsdp(mods, plugin)
    assert len(plugin.ignored_modules) == 4
    for m in mods:
        assert all(getattr(p, "_fmsb_replicated", False) for p in m.lora_A.parameters())
        assert all(getattr(p, "_fmsb_replicated", False) for p in m.lora_B.parameters())
        assert not hasattr(m.base_layer.weight, "_fmsb_replicated")
