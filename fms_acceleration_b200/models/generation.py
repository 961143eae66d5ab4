"""Token generation for the in-tree causal language models: what ``model.generate`` offers on a Hugging Face model,
which the reference's GPTQ wrapper forwards to (fms_acceleration_peft/gptqmodel/models/base.py:539-546).

The models of this package are training models: their attention kernels take whole (packed) sequences and keep no
key / value cache.  Generation therefore runs the whole prefix again for every new token; it is meant for checking a
fine-tuned model on a few prompts, not for serving."""
from __future__ import annotations

from typing import Optional

import torch


class GenerationMixin:
    def prepare_inputs_for_generation(self, input_ids, **kwargs):
        """The keyword arguments of one forward during generation (no cache: always the whole prefix)."""
        return {"input_ids": input_ids, "return_logits": True}

    @torch.no_grad()
    def generate(self, input_ids: Optional[torch.Tensor] = None, max_new_tokens: int = 20, max_length: Optional[int] = None,
                 do_sample: bool = False, temperature: float = 1.0, top_k: Optional[int] = None,
                 top_p: Optional[float] = None, eos_token_id: Optional[int] = None, pad_token_id: Optional[int] = None,
                 generator: Optional[torch.Generator] = None, **kwargs) -> torch.Tensor:
        """``input_ids [B, S]`` (rows of equal length, no padding) -> ``[B, S + new]``.  Greedy unless ``do_sample``
        (then temperature / top-k / top-p sampling).  A row that has produced ``eos_token_id`` is filled with
        ``pad_token_id`` (default: the end token) from then on; generation stops when every row has ended."""
        if input_ids is None:
            raise ValueError("generate() needs input_ids")
        if input_ids.dim() == 1:
            input_ids = input_ids[None]
        if max_length is not None:
            max_new_tokens = max(0, max_length - input_ids.shape[1])
        pad = pad_token_id if pad_token_id is not None else eos_token_id
        was_training = self.training
        self.eval()
        try:
            ids = input_ids
            done = torch.zeros(ids.shape[0], dtype=torch.bool, device=ids.device)
            for _ in range(max_new_tokens):
                out = self(**self.prepare_inputs_for_generation(ids))
                logits = (out.logits if hasattr(out, "logits") else out[0])[:, -1].float()
                if do_sample:
                    nxt = _sample(logits, temperature, top_k, top_p, generator)
                else:
                    nxt = logits.argmax(-1)
                if eos_token_id is not None:
                    nxt = torch.where(done, torch.full_like(nxt, pad), nxt)
                    done = done | (nxt == eos_token_id)
                ids = torch.cat([ids, nxt[:, None].to(ids.dtype)], dim=1)
                if eos_token_id is not None and bool(done.all()):
                    break
            return ids
        finally:
            self.train(was_training)


def _sample(logits, temperature, top_k, top_p, generator):
    logits = logits / max(float(temperature), 1e-6)
    if top_k is not None and 0 < top_k < logits.shape[-1]:
        kth = torch.topk(logits, top_k, dim=-1).values[:, -1:]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    if top_p is not None and 0.0 < top_p < 1.0:
        sorted_logits, order = torch.sort(logits, descending=True, dim=-1)
        probs = torch.softmax(sorted_logits, -1)
        # keep the smallest set of tokens whose probability mass reaches top_p (the first token always stays)
        drop = probs.cumsum(-1) - probs > top_p
        sorted_logits = sorted_logits.masked_fill(drop, float("-inf"))
        logits = torch.full_like(logits, float("-inf")).scatter(-1, order, sorted_logits)
    return torch.multinomial(torch.softmax(logits, -1), 1, generator=generator).squeeze(-1)
