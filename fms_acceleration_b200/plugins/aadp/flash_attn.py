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
