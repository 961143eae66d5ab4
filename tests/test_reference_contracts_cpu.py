"""Behaviour that the reference's own CPU test-suites pin down and that differed here before those suites were run
against the alias packages: a model without a config is an error at augmentation, streaming category datasets feed
the mixing dataset, the auto-categoriser's module-level embedder name / input checks, and the test utilities being
importable from ``fms_acceleration.utils``."""
import numpy as np
import pytest
import torch


def test_test_utilities_are_exported_by_the_utils_package():
    from fms_acceleration.utils import (build_framework_and_maybe_instantiate, create_noop_model_with_archs,  # noqa: F401
                                        create_plugin_cls, instantiate_framework, read_configuration)
    from fms_acceleration.utils.test_utils import instantiate_framework as direct

    assert instantiate_framework is direct


def test_augmentation_of_a_model_without_config_is_an_attribute_error():
    from fms_acceleration.utils import build_framework_and_maybe_instantiate, create_plugin_cls

    plugin = create_plugin_cls(requires_augmentation=True)
    with build_framework_and_maybe_instantiate([(["dummy"], plugin)], configuration_contents={"dummy": {"key1": 1}},
                                               instantiate=True) as framework:
        with pytest.raises(AttributeError):
            framework.augmentation(torch.nn.Module(), None, None)


class _Stream(torch.utils.data.IterableDataset):
    """Endless stream of samples without a usable ``len``."""

    def __init__(self, value):
        self.value = value

    def __len__(self):
        return None  # what a streaming dataset without a length amounts to

    def __iter__(self):
        n = 0
        while True:
            yield {"input_ids": torch.full((4,), self.value + n)}
            n += 1


def test_streaming_categories_feed_the_mixing_dataset_and_resume(tmp_path):
    from fms_acceleration_odm import OnlineMixingDataset, Reward

    data = {"a": _Stream(0), "b": _Stream(100)}
    ds = OnlineMixingDataset(data, {"a": None, "b": None}, data, {"a": None, "b": None}, {"a": 1, "b": 1}, 0.1, 0.3, 1,
                             2, output_dir=str(tmp_path), reward_type=Reward.ENTROPY)
    seen = {"a": [], "b": []}
    for _ in range(12):
        sample = next(ds)
        cat = ds.id2cat[ds.arm_idx]
        seen[cat].append(int(sample["input_ids"].reshape(-1)[0]))
    # every category's stream is consumed in order, one sample at a time
    assert seen["a"] == list(range(len(seen["a"]))) and seen["b"] == [100 + i for i in range(len(seen["b"]))]
    # a restored position skips what was already consumed
    loader = ds.train_dataset_dict_dl["a"]
    state = loader.state_dict()
    loader.load_state_dict(state)
    assert int(next(loader)["input_ids"].reshape(-1)[0]) == len(seen["a"])


class _FakeEmbedder:
    def __init__(self, *args, **kwargs):
        self.kwargs = kwargs

    def encode(self, texts, **_):
        # two well separated groups by the parity of the text's length
        return np.asarray([[0.0, 0.0] if len(t) % 2 == 0 else [10.0, 10.0] for t in texts], dtype=np.float32)


class _Table:
    """The few members of a Hugging Face ``Dataset`` the categoriser uses."""

    def __init__(self, columns):
        self.columns = columns
        self.column_names = list(columns)

    def __len__(self):
        return len(next(iter(self.columns.values())))

    def __getitem__(self, key):
        if isinstance(key, str):
            return self.columns[key]
        return {k: v[key] for k, v in self.columns.items()}

    def select(self, idx):
        return _Table({k: [v[i] for i in idx] for k, v in self.columns.items()})


def test_auto_categoriser_contract(monkeypatch):
    from fms_acceleration_odm.odm import auto_categorizer as AC

    monkeypatch.setattr("fms_acceleration_odm.odm.auto_categorizer.SentenceTransformer", _FakeEmbedder)
    table = _Table({"text": ["aa", "bbb", "cc", "ddd", "ee", "fff"]})
    out = AC.DatasetAutoCategorizer(AC.AutoCategorizeConfig(num_categories=2, category_prefix="cluster"))(table)
    assert set(out) == {"cluster_0", "cluster_1"} and sum(len(v) for v in out.values()) == 6
    assert {tuple(sorted(v["text"])) for v in out.values()} == {("aa", "cc", "ee"), ("bbb", "ddd", "fff")}

    with pytest.raises(ValueError, match="missing column"):
        AC.DatasetAutoCategorizer(AC.AutoCategorizeConfig(input_column="content"))(table)
    with pytest.raises(ValueError, match="empty"):
        AC.DatasetAutoCategorizer()(_Table({"text": []}))
    with pytest.raises(NotImplementedError, match="not yet supported"):
        AC.DatasetAutoCategorizer()(_Stream(0))

    tokens = _Table({"input_ids": [[1, 2], [3, 4, 5], [6, 7], [8, 9, 10]]})
    with pytest.raises(AssertionError):  # token ids and no tokenizer to turn them back into text
        AC.DatasetAutoCategorizer(AC.AutoCategorizeConfig(input_column="input_ids", num_categories=2))(tokens)

    class Tok:
        def batch_decode(self, rows):
            return ["x" * len(r) for r in rows]

    cfg = AC.AutoCategorizeConfig(input_column="input_ids", num_categories=2, tokenizer=Tok())
    out = AC.DatasetAutoCategorizer(cfg)(tokens)
    assert sorted(len(v) for v in out.values()) == [2, 2] and cfg.input_column == "input_ids"

    # category count: the given number, else floor(sqrt(n)) inside [min, max], never more than rows
    count = AC.DatasetAutoCategorizer(AC.AutoCategorizeConfig())._num_clusters
    assert count(3) == 2 and count(30) == 5 and count(10 ** 6) == 15 and count(1) == 1
    assert AC.DatasetAutoCategorizer(AC.AutoCategorizeConfig(num_categories=40))._num_clusters(100) == 40
