"""``generate`` of the in-tree causal language models: greedy decoding equals the arg-max loop written out, sampling
honours top-k, and rows that have ended are padded."""
import pytest
import torch

from fms_acceleration_b200.models.builder import build_model


@pytest.mark.parametrize("preset,rows", [("tiny-llama", 2), ("tiny-gpt-bigcode", 2), ("tiny-mamba2", 1),
                                         ("tiny-granitemoe", 2), ("tiny-granitemoehybrid", 1)])
def test_greedy_generation_is_the_argmax_loop(preset, rows):
    torch.manual_seed(0)
    model = build_model(preset, device="cpu", dtype=torch.float32)
    ids = torch.randint(0, model.config.vocab_size, (rows, 5))
    out = model.generate(ids, max_new_tokens=3)
    want = ids
    with torch.no_grad():
        for _ in range(3):
            nxt = model(want, return_logits=True).logits[:, -1].argmax(-1)
            want = torch.cat([want, nxt[:, None]], dim=1)
    assert torch.equal(out, want)
    assert model.training  # the mode the model was in is restored
    assert model.generate(ids, max_length=7).shape == (rows, 7)


def test_sampling_and_end_of_sequence():
    torch.manual_seed(1)
    model = build_model("tiny-llama", device="cpu", dtype=torch.float32)
    ids = torch.randint(0, model.config.vocab_size, (2, 4))
    with torch.no_grad():
        logits = model(ids, return_logits=True).logits[:, -1]
    allowed = torch.topk(logits, 3, dim=-1).indices
    for seed in range(5):
        out = model.generate(ids, max_new_tokens=1, do_sample=True, top_k=3, temperature=0.8,
                             generator=torch.Generator().manual_seed(seed))
        assert all(int(out[r, -1]) in allowed[r].tolist() for r in range(2))
    one = model.generate(ids, max_new_tokens=1, do_sample=True, top_p=1e-6, generator=torch.Generator().manual_seed(0))
    assert torch.equal(one[:, -1], logits.argmax(-1))  # a vanishing nucleus keeps only the most likely token

    greedy = model.generate(ids, max_new_tokens=4)
    eos = int(greedy[0, 4])  # the first token row 0 produces
    out = model.generate(ids, max_new_tokens=4, eos_token_id=eos, pad_token_id=7)
    assert int(out[0, 4]) == eos and out[0, 5:].tolist() == [7] * (out.shape[1] - 5)
    single = model.generate(ids[:1], max_new_tokens=4, eos_token_id=eos)
    assert single.shape[1] == 5  # stops as soon as every row has ended
