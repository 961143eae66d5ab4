"""Adapter from Hugging Face's ``_flash_attention_forward`` call convention to the in-tree varlen kernel
(role of fms_acceleration_aadp/flash_attn.py:36-199 in the reference: derive ``cu_seqlens`` from the places
where ``position_ids == 0`` and call a varlen attention)."""
from __future__ import annotations

import torch

from ...ops.attention import cu_seqlens_from_position_ids, doc_bounds_from_cu_seqlens, varlen_attention


def prepare_fa2_from_position_ids(query, key, value, position_ids):
    """Flatten ``[B, S, heads, d]`` tensors to ``[B*S, heads, d]`` and derive the document boundaries."""
    q = query.reshape(-1, query.size(-2), query.size(-1))
    k = key.reshape(-1, key.size(-2), key.size(-1))
    v = value.reshape(-1, value.size(-2), value.size(-1))
    cu = cu_seqlens_from_position_ids(position_ids)
    return q, k, v, cu


#: position ids of the batch a model is processing, by model id: older transformers versions do not hand the position
#: ids to the attention function, the backbone's forward leaves them here (as in the reference, flash_attn.py:33-82)
POSITION_IDS_CACHE: dict = {}


def build_backbone_forward(model: torch.nn.Module, model_id: str):
    """A ``forward`` for the decoder backbone that records the batch's ``position_ids`` under ``model_id`` before
    calling the original one.  Meant to be bound as a method (first argument ``self``)."""
    original = model.forward

    def forward(self, *args, **kwargs):
        POSITION_IDS_CACHE[model_id] = kwargs.get("position_ids")
        return original(*args, **kwargs)

    return forward


def build_fa_forward():
    def _flash_attention_forward(query_states, key_states, value_states, attention_mask=None, query_length=None,
                                 is_causal=True, dropout=0.0, position_ids=None, softmax_scale=None, **kwargs):
        B, S = query_states.shape[0], query_states.shape[1]
        if position_ids is None:
            position_ids = torch.arange(S, device=query_states.device).expand(B, S)
        q, k, v, cu = prepare_fa2_from_position_ids(query_states, key_states, value_states, position_ids)
        ds, de = doc_bounds_from_cu_seqlens(cu, q.shape[0])
        out = varlen_attention(q, k, v, ds, de, softmax_scale)
        return out.view(B, S, out.shape[1], out.shape[2])

    return _flash_attention_forward


# ---------------------------------------------------------------------------------------------------------
# transformers >= 4.48 dispatches attention through a registry (``config._attn_implementation`` -> function).
# The in-tree kernel is registered there under its own name, so a Hugging Face model uses it without any
# flash-attn package and without touching the modeling code.
# ---------------------------------------------------------------------------------------------------------
HF_ATTENTION_NAME = "fmsb_varlen"
_BOUNDS_CACHE: dict = {}


def _doc_bounds(position_ids, cu_seq_lens, total: int, device):
    """Document start / end per row of the flattened batch; computed once per batch, not once per layer.  The cache
    holds a weak reference to the tensor object the layers of one forward pass share: a later batch is a different
    object even when the allocator hands it the same address."""
    import weakref

    src = cu_seq_lens if cu_seq_lens is not None else position_ids
    hit = _BOUNDS_CACHE.get("last")
    if hit is not None and hit[0]() is src and hit[1] == (src._version, total):
        return hit[2]
    cu = cu_seq_lens.to(torch.int32) if cu_seq_lens is not None else cu_seqlens_from_position_ids(position_ids)
    bounds = doc_bounds_from_cu_seqlens(cu.to(device), total)
    _BOUNDS_CACHE["last"] = (weakref.ref(src), (src._version, total), bounds)
    return bounds


def hf_attention_forward(module, query, key, value, attention_mask, dropout: float = 0.0, scaling=None,
                         sliding_window=None, softcap=None, is_causal=None, **kwargs):
    """Attention-interface function: ``query [B, heads, S, d]``, ``key``/``value [B, kv heads, S, d]`` ->
    ``([B, S, heads, d], None)``.  Documents are delimited by ``cu_seq_lens_q`` when the collator provides it, else
    by the zeros of ``position_ids``, else every row of the batch is one document."""
    B, nh, S, d = query.shape
    if softcap is not None:
        raise NotImplementedError("logit soft-capping is not supported by the varlen attention kernel")
    if sliding_window is not None and sliding_window < S:
        raise NotImplementedError("sliding-window attention shorter than the sequence is not supported")
    if attention_mask is not None and attention_mask.dim() == 2 and not bool(attention_mask.all()):
        raise NotImplementedError("padded batches are not supported: use the padding-free collator")
    if key.shape[2] != S:
        raise NotImplementedError("the varlen attention kernel is for training (no key/value cache)")
    q = query.transpose(1, 2).reshape(B * S, nh, d).contiguous()
    k = key.transpose(1, 2).reshape(B * S, key.shape[1], d).contiguous()
    v = value.transpose(1, 2).reshape(B * S, value.shape[1], d).contiguous()
    position_ids, cu_q = kwargs.get("position_ids"), kwargs.get("cu_seq_lens_q")
    if position_ids is None and cu_q is None:
        # no packing information: every row of the batch is one document
        cu_q = torch.arange(0, (B + 1) * S, S, dtype=torch.int32, device=query.device)
        ds, de = doc_bounds_from_cu_seqlens(cu_q, B * S)
    else:
        ds, de = _doc_bounds(position_ids, cu_q, B * S, query.device)
    out = varlen_attention(q, k, v, ds, de, scaling)
    return out.view(B, S, nh, d), None


def register_hf_attention() -> bool:
    """Register :func:`hf_attention_forward` (and a mask function that builds no dense mask) with transformers'
    attention registry.  Returns False when the installed transformers has no such registry."""
    try:
        from transformers import AttentionInterface
        from transformers.masking_utils import ALL_MASK_ATTENTION_FUNCTIONS, AttentionMaskInterface
    except Exception:
        return False
    AttentionInterface.register(HF_ATTENTION_NAME, hf_attention_forward)
    AttentionMaskInterface.register(HF_ATTENTION_NAME, ALL_MASK_ATTENTION_FUNCTIONS["flash_attention_2"])
    return True


def use_in_tree_attention(model) -> bool:
    """Point a Hugging Face model (also through a PEFT wrapper) at the registered attention function."""
    if not register_hf_attention():
        return False
    seen = False
    for m in model.modules():
        cfg = getattr(m, "config", None)
        if cfg is not None and hasattr(cfg, "_attn_implementation"):
            cfg._attn_implementation = HF_ATTENTION_NAME
            seen = True
    return seen
