"""Online data mixing: EXP3 arithmetic, learning, state round trip, rewards, plugin behaviour."""
import json
import math
import os

import pytest
import torch

from fms_acceleration_b200.plugins.odm import OnlineMixingDataset, Reward, compute_reward
from fms_acceleration_b200.plugins.odm.odm import reward as R
from fms_acceleration_b200.plugins.odm.odm.auto_categorizer import AutoCategorizeConfig, DatasetAutoCategorizer


class _DS(list):
    pass


def _make(tmp_path, **kw):
    cats = {c: _DS({"input_ids": torch.tensor([i, i + 1, i + 2])} for i in range(base, base + 7))
            for c, base in (("a", 0), ("b", 100), ("c", 200))}
    return OnlineMixingDataset(cats, None, {c: None for c in cats}, None, output_dir=str(tmp_path), **kw)


def test_exp3_ratio_and_update(tmp_path):
    ds = _make(tmp_path, gamma=0.2, eta=0.5)
    assert ds.sampling_ratio == pytest.approx([1 / 3] * 3)
    ratio_before = list(ds.sampling_ratio)
    ds._update_weights([2, 2, 2], [1.0, 0.0, 4.0])
    w = [math.exp(0.5 * (r / 2 / ratio_before[i]) / 3) for i, r in enumerate([1.0, 0.0, 4.0])]
    exp_ratio = [(1 - 0.2) * wi / sum(w) + 0.2 / 3 for wi in w]
    assert ds.sampling_ratio == pytest.approx(exp_ratio)
    assert ds.sampling_ratio[2] > ds.sampling_ratio[0] > ds.sampling_ratio[1]


def test_sampling_is_seeded_logged_and_resumable(tmp_path):
    a, b = _make(tmp_path / "x", seed=7), _make(tmp_path / "y", seed=7)
    seq_a = [next(a)["input_ids"].tolist() for _ in range(20)]
    seq_b = [next(b)["input_ids"].tolist() for _ in range(20)]
    assert seq_a == seq_b  # every rank draws the same order
    assert sum(a.curr_cat_count) == 20 and a.produced == 20
    lines = open(a.log_file_path).read().strip().splitlines()
    assert len(lines) == 20 and json.loads(lines[-1])["action"] == "sample"
    assert os.path.basename(a.log_file_path) == "odm_rank_0.jsonl"
    state = a.state_dict()
    cont = [next(a)["input_ids"].tolist() for _ in range(15)]
    c = _make(tmp_path / "z", seed=7)
    c.load_state_dict(state)
    assert [next(c)["input_ids"].tolist() for _ in range(15)] == cont


def test_bandit_learns_the_rewarding_arm(tmp_path):
    ds = _make(tmp_path, gamma=0.1, eta=0.3)
    for _ in range(60):
        ds._update_weights([1, 1, 1], [0.05, 0.9, 0.05])
    assert ds.sampling_ratio[1] > 0.8


class _Out:
    def __init__(self, logits):
        self.logits = logits


class _Uniform(torch.nn.Module):
    def forward(self, input_ids=None, attention_mask=None, labels=None):
        return _Out(torch.zeros(*input_ids.shape, 16))


class _Peaked(torch.nn.Module):
    def forward(self, input_ids=None, attention_mask=None, labels=None):
        lg = torch.full((*input_ids.shape, 16), -50.0)
        lg[..., 0] = 50.0
        return _Out(lg)


def test_entropy_rewards():
    batch = {"input_ids": torch.ones(3, 6, dtype=torch.long), "attention_mask": torch.ones(3, 6, dtype=torch.long)}
    assert compute_reward(_Uniform(), batch, 16, Reward.ENTROPY) == pytest.approx(3.0, abs=1e-4)
    assert compute_reward(_Peaked(), batch, 16, "entropy") == pytest.approx(0.0, abs=1e-4)
    assert compute_reward(_Uniform(), batch, 16, Reward.ENTROPY_LAST_TOKEN) == pytest.approx(3.0, abs=1e-4)
    assert compute_reward(_Uniform(), batch, 16, Reward.ENTROPY3_VARENT1) == pytest.approx(0.75 * 3.0, abs=1e-3)


def test_history_rewards():
    R.TRAIN_LOSS_DATA["buffer"], R.GRADNORM_DATA["buffer"], R.EVAL_LOSS_DATA["buffer"] = [], [], []
    r = compute_reward(None, None, 16, Reward.TRAIN_LOSS, train_loss_history=[{"loss": 2.5}], last_sampled_category=1,
                       total_categories=3, current_category=1)
    assert r == 2.5
    assert compute_reward(None, None, 16, Reward.TRAIN_LOSS, train_loss_history=[{"loss": 2.5}], last_sampled_category=1,
                          total_categories=3, current_category=0) == pytest.approx(1e-100)
    g = compute_reward(None, None, 16, Reward.GRADNORM, gradnorm_history=[{"grad_norm": 4.0}], last_sampled_category=2,
                       total_categories=3, current_category=2)
    assert g == pytest.approx(1 / 4.0001)
    with pytest.raises(ValueError):
        compute_reward(None, None, 16, Reward.VALIDATION_LOSS, eval_loss_history=[], total_categories=3, current_category=0)
    with pytest.raises(ValueError):
        Reward.parse("nonsense")


def test_update_sampling_weights_with_model(tmp_path):
    cats = {"a": _DS({"input_ids": torch.tensor([1, 2, 3])} for _ in range(4)),
            "b": _DS({"input_ids": torch.tensor([4, 5, 6])} for _ in range(4))}
    evals = {c: [{"input_ids": torch.tensor([1, 2, 3, 4]), "attention_mask": torch.ones(4, dtype=torch.long)}
                 for _ in range(4)] for c in cats}
    ds = OnlineMixingDataset(cats, None, evals, None, output_dir=str(tmp_path), eval_batch_size=2, vocab_size=16)
    ds.update_sampling_weights(_Uniform(), None, None)
    last = json.loads(open(ds.log_file_path).read().strip().splitlines()[-1])
    assert last["action"] == "update" and last["count"] == [4, 4]
    assert last["rewards"] == pytest.approx([4.0, 4.0], abs=1e-3)


def test_auto_categorizer_with_stub_embedder(monkeypatch):
    class Data(list):
        column_names = ["text"]

        def __getitem__(self, k):
            return [r["text"] for r in self] if k == "text" else list.__getitem__(self, k)

        def select(self, idx):
            return Data(list.__getitem__(self, i) for i in idx)

    data = Data({"text": t} for t in ["aa"] * 10 + ["zz"] * 10)
    cat = DatasetAutoCategorizer(AutoCategorizeConfig(num_categories=2))
    monkeypatch.setattr(cat, "_embed", lambda texts: torch.tensor([[1.0, 0.0] if t == "aa" else [0.0, 1.0]
                                                                   for t in texts]).numpy())
    out = cat(data)
    assert sorted(len(v) for v in out.values()) == [10, 10] and all(k.startswith("auto_category_") for k in out)


def test_plugin_rewrites_eval_schedule(tmp_path):
    from fms_acceleration_b200.framework.utils.test_utils import instantiate_framework, read_configuration
    from fms_acceleration_b200.trainer import TrainArgs
    import fms_acceleration_b200.plugins as P

    cfg = read_configuration(os.path.join(os.path.dirname(P.__file__), "odm", "configs", "odm.yaml"))
    with instantiate_framework(cfg) as fw:
        assert [n for n, _ in fw.active_plugins] == ["OnlineDataMixingAccelerationPlugin"]
        model = torch.nn.Linear(2, 2)
        model.config = type("C", (), {"architectures": ["X"]})
        args = TrainArgs(eval_steps=50)
        fw.augmentation(model, args, modifiable_args=(None,))
        assert model.ta_eval_steps == 50 and args.eval_steps == 1 and args.eval_strategy == "steps"
        assert model.ta_update_interval == 1


def test_custom_training_loop_example_runs(capsys):
    """The hand-written loop of the artifacts folder (mixing dataset + plain DataLoader + periodic bandit update)."""
    from fms_acceleration_b200.plugins.odm.artifacts import custom_loop_usage

    assert custom_loop_usage.main(["--steps", "12", "--batch", "2"]) == 0
    out = capsys.readouterr().out
    assert "step 10:" in out and "sampling ratio" in out
