"""``ScatterMoE`` module: drop-in replacement of a Hugging Face sparse-MoE block.

Parameter names and layout follow the reference (fms_acceleration_moe/utils/scattermoe.py:44-491): ``router``
(``nn.Linear``, weight ``[E, H]``), ``w1`` / ``w3`` (``ScatteredExperts`` with ``weight [E, H, I]``) and ``w2``
(``weight [E, I, H]``); ``forward`` returns ``(hidden_states, router_logits)``.  With expert parallelism a rank
holds the ``E / ep`` experts ``[rank * E/ep, (rank + 1) * E/ep)``.  Execution is
:mod:`fms_acceleration_b200.ops.moe` (device-side plan, peer-memory dispatch / combine, grouped tcgen05 GEMMs).
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.nn.functional as F
from torch import nn

from ....ops import moe as MOE


class ScatteredExperts(nn.Module):
    def __init__(self, in_features: int, out_features: int, num_experts: int, fan_out: int = 1, grouped_in: bool = False,
                 grouped_out: bool = False, dtype=torch.bfloat16, device=None, lora_config=None):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(num_experts, in_features, out_features, dtype=dtype, device=device))
        self.in_features, self.out_features, self.num_experts = in_features, out_features, num_experts
        self.fan_out, self.grouped_in, self.grouped_out = fan_out, grouped_in, grouped_out
        self.lora_A = self.lora_B = None
        self.lora_r = 0
        if lora_config is not None:
            r = lora_config.r
            self.lora_r = r
            self.weight.requires_grad_(False)
            self.lora_A = nn.Parameter(torch.zeros(num_experts, in_features, r, dtype=dtype, device=device))
            self.lora_B = nn.Parameter(torch.empty(num_experts, r, out_features, dtype=dtype, device=device))
            nn.init.normal_(self.lora_B)

    def effective_weight(self) -> torch.Tensor:
        """Dense expert weights including the LoRA update (scale 1, as in the reference's kernels).  Used by the
        library / CPU paths and as the oracle of the fused path, which never forms it."""
        if self.lora_A is None:
            return self.weight
        return self.weight + torch.bmm(self.lora_A, self.lora_B)

    def forward(self, x, bin_ids, indices, padded_block_idxs, expert_offsets, gates=None):
        """One projection on its own, rows gathered into expert order on the way in and scattered back on the way out
        (the reference's ``ScatteredExperts.forward``, fms_acceleration_moe/utils/scattermoe.py:129-181).
        ``bin_ids``: sorted expert of every (token, choice) pair; ``indices``: the permutation that sorts the pairs;
        ``expert_offsets``: where each expert's rows end; ``gates [T, k]``: weights of the sum over a token's rows.
        ``ScatterMoE.forward`` does not call this: it runs both projections and the combine as one fused operator."""
        from .scattermoe_utils.khd.kernels.ops import scattered_experts

        return scattered_experts(x, self.weight, self.fan_out, bin_ids, indices, padded_block_idxs, expert_offsets,
                                 gates=gates, grouped_in=self.grouped_in, grouped_out=self.grouped_out,
                                 expert_lora_A=self.lora_A, expert_lora_B=self.lora_B, lora_alp=float(self.lora_r))


class ScatterMoE(nn.Module):
    def __init__(self, hidden_size: int, hidden_act: str, intermediate_size: int, num_experts: int,
                 has_bias: bool = False, mlp_arch: Optional[str] = None, top_k: int = 2, dtype=torch.bfloat16,
                 device=None, ep_device_mesh=None, ep_group=None, lora_config=None, token_budget: Optional[int] = None):
        super().__init__()
        assert not has_bias, "ScatterMoE does not support bias"
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.num_experts, self.top_k = num_experts, top_k
        self.activation = hidden_act
        if ep_device_mesh is not None and ep_group is None:
            ep_group = ep_device_mesh.get_group(0) if hasattr(ep_device_mesh, "get_group") else None
        self.ep_group = ep_group
        self.expert_parallel = ep_group is not None
        self.ep_size = torch.distributed.get_world_size(ep_group) if self.expert_parallel else 1
        assert num_experts % self.ep_size == 0, "the expert-parallel degree must divide the number of experts"
        self.num_experts_per_device = num_experts // self.ep_size
        self.router = nn.Linear(hidden_size, num_experts, bias=False, dtype=dtype, device=device)
        El = self.num_experts_per_device
        self.w1 = ScatteredExperts(hidden_size, intermediate_size, El, top_k, grouped_out=True, dtype=dtype, device=device,
                                   lora_config=lora_config)
        self.w2 = ScatteredExperts(intermediate_size, hidden_size, El, 1, grouped_in=True, dtype=dtype, device=device,
                                   lora_config=lora_config)
        self.w3 = ScatteredExperts(hidden_size, intermediate_size, El, top_k, grouped_out=True, dtype=dtype, device=device,
                                   lora_config=lora_config)
        # largest number of tokens this rank hands to one forward (sizes the expert-parallel staging once)
        self.token_budget = token_budget
        self._ctx: Optional[MOE.MoEContext] = None
        # "fused": this package's kernels (peer-memory dispatch / combine around grouped tcgen05 GEMMs).
        # "library": torch ops and, under expert parallelism, all_to_all_single of the process group's backend
        # (NCCL on GPUs, gloo on CPUs): the like-for-like baseline of the fused path and the CPU execution path.
        self.backend = os.environ.get("FMSB_MOE_BACKEND", "fused")

    def _context(self) -> MOE.MoEContext:
        if self._ctx is None:
            self._ctx = MOE.MoEContext(self.hidden_size, self.intermediate_size, self.num_experts, self.top_k,
                                       group=self.ep_group, token_budget=self.token_budget)
        return self._ctx

    def _compute_routing_weights(self, x2: torch.Tensor):
        if x2.is_cuda and x2.dtype in (torch.bfloat16, torch.float16):
            from ....models.llama import _DenseLinear

            logits = _DenseLinear.apply(x2, self.router.weight)
        else:
            logits = self.router(x2)
        w, idx = MOE.router_topk(logits, self.top_k, renorm=True)
        return logits, w, idx

    def forward(self, hidden_states: torch.Tensor):
        shape = hidden_states.shape
        x2 = hidden_states.reshape(-1, shape[-1])
        if x2.stride(1) != 1 or x2.stride(0) % 8:
            x2 = x2.contiguous()
        logits, w, idx = self._compute_routing_weights(x2)
        if x2.is_cuda and x2.dtype in (torch.bfloat16, torch.float16) and self.backend == "fused":
            lora = None
            if self.w1.lora_A is not None:
                # frozen expert weights plus per-expert low-rank factors: the low-rank products ride in the grouped
                # GEMMs as a second operand pair, the dense W + A B is never formed
                lora = MOE.pack_expert_lora(self.w1.lora_A, self.w1.lora_B, self.w3.lora_A, self.w3.lora_B,
                                            self.w2.lora_A, self.w2.lora_B)
            out = MOE.experts_forward(x2, w, idx, self.w1.weight, self.w3.weight, self.w2.weight, self._context(),
                                      self.activation, lora=lora)
        elif self.expert_parallel:
            out = self._forward_library_ep(x2, w, idx)
        else:
            out = self._forward_reference(x2, w, idx)
        return (out.view(shape), logits) if getattr(self, "return_router_logits", True) else out.view(shape)

    def _forward_library_ep(self, x2, w, idx):
        """Expert parallelism with library collectives (the exchange of the reference,
        fms_acceleration_moe/utils/scattermoe_utils/expert_parallel.py:97-232): rows sorted by expert, counts and
        rows exchanged with all-to-all (one host synchronisation for the split sizes), local experts as dense
        matmuls per expert, rows sent back and summed with the routing weights."""
        from .scattermoe_utils import all_to_all_gather_inputs, scatter_with_routing_weights

        El = self.num_experts_per_device
        rows, local_e, state = all_to_all_gather_inputs(x2, idx, self.ep_group, self.top_k, El)
        w1, w2, w3 = (m.effective_weight() for m in (self.w1, self.w2, self.w3))
        act = {"silu": F.silu, "gelu": F.gelu}.get(self.activation, F.silu)
        counts = torch.bincount(local_e, minlength=El).tolist()  # rows arrive ordered by local expert
        outs, start = [], 0
        for e in range(El):
            xe = rows[start:start + counts[e]]
            start += counts[e]
            outs.append((act(xe @ w1[e]) * (xe @ w3[e])) @ w2[e])
        y = torch.cat(outs) if outs else rows.new_zeros(0, x2.shape[1])
        return scatter_with_routing_weights(y, w, state).to(x2.dtype)

    def _forward_reference(self, x2, w, idx):
        out = torch.zeros_like(x2, dtype=torch.float32)
        w1, w2, w3 = (m.effective_weight().float() for m in (self.w1, self.w2, self.w3))
        act = {"silu": F.silu, "gelu": F.gelu}.get(self.activation, F.silu)
        xf = x2.float()
        for e in range(self.num_experts):
            tok, slot = torch.nonzero(idx == e, as_tuple=True)
            if tok.numel() == 0:
                continue
            h = act(xf[tok] @ w1[e]) * (xf[tok] @ w3[e])
            out.index_add_(0, tok, (h @ w2[e]) * w[tok, slot][:, None].float())
        return out.to(x2.dtype)
