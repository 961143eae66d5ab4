"""Pseudo-categories for a single un-labelled dataset: embed every sample, cluster with k-means, one category per
cluster (role of fms_acceleration_odm/odm/auto_categorizer.py:38-201).  The embedding model (sentence-transformers)
and cuML are optional; scikit-learn's KMeans is the default clusterer."""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import numpy as np
import torch

try:  # optional dependency; the module-level name is what callers (and tests) may replace
    from sentence_transformers import SentenceTransformer
except ImportError:  # pragma: no cover - depends on the environment
    SentenceTransformer = None

#: column that receives the rebuilt text of a pre-tokenised dataset
AUTO_CATEGORIZATION_COLUMN_NAME = "auto_categorization_text"


@dataclass
class AutoCategorizeConfig:
    input_column: str = "text"
    num_categories: Optional[int] = None        # default: round(sqrt(N)) clamped to [min_categories, max_categories]
    min_categories: int = 2
    max_categories: int = 15
    model_name: str = "Qwen/Qwen3-Embedding-0.6B"
    batch_size: int = 64
    category_prefix: str = "auto_category"
    tokenizer: Any = None                       # when given, ``input_ids`` are detokenised into text first
    seed: int = 42
    model_kwargs: Dict[str, Any] = field(default_factory=dict)
    cluster_algo: str = "kmeans"                # the only clustering offered, as in the reference
    cluster_kwargs: Dict[str, Any] = field(default_factory=dict)   # extra arguments of the clusterer
    kmeans_kwargs: Dict[str, Any] = field(default_factory=dict)    # older name of ``cluster_kwargs``; both apply


class DatasetAutoCategorizer:
    def __init__(self, config: Optional[AutoCategorizeConfig] = None):
        # a private copy: a pre-tokenised dataset redirects ``input_column`` to the rebuilt text
        self.config = copy.copy(config) if config is not None else AutoCategorizeConfig()

    # -- pieces ---------------------------------------------------------------------------------------
    def _column(self, dataset, name: str):
        cols = getattr(dataset, "column_names", None)
        if cols is not None:
            return dataset[name]
        return [dataset[i][name] for i in range(len(dataset))]

    def _texts(self, dataset) -> List[str]:
        """The strings to embed: the input column itself, or, when it holds token ids, their decoding (which needs
        ``config.tokenizer``; an AssertionError without one, as in the reference :107-135)."""
        c = self.config
        cols = getattr(dataset, "column_names", None)
        if cols is None:
            cols = list(dataset[0].keys())
        if c.input_column not in cols:
            raise ValueError(f"Dataset is missing column '{c.input_column}'. Provide a input field in "
                             "auto_categorize_config['input_column'].")
        values = self._column(dataset, c.input_column)
        if isinstance(values[0], str):
            return [str(t) for t in values]
        assert c.tokenizer is not None, (
            f"Attempting detokenizing the data on column '{c.input_column}' but the tokenizer is not provided")
        assert AUTO_CATEGORIZATION_COLUMN_NAME not in cols, (
            f"Default detokenizing column '{AUTO_CATEGORIZATION_COLUMN_NAME}' is already present in the dataset")
        rows = [v.tolist() if hasattr(v, "tolist") else list(v) for v in values]
        if hasattr(c.tokenizer, "batch_decode"):
            return list(c.tokenizer.batch_decode(rows))
        return [c.tokenizer.decode(r) for r in rows]

    def _embed(self, texts: List[str]) -> np.ndarray:
        if SentenceTransformer is None:
            raise ImportError("auto-categorisation needs the sentence-transformers package for its embeddings")
        model = SentenceTransformer(self.config.model_name, model_kwargs=self.config.model_kwargs,
                                    prompts={"clustering": "Identify the topic or theme based on the text: "},
                                    default_prompt_name="clustering")
        emb = model.encode(texts, batch_size=self.config.batch_size, convert_to_numpy=True, normalize_embeddings=True,
                           show_progress_bar=False)
        return np.asarray(emb, dtype=np.float32)

    def _num_clusters(self, n: int) -> int:
        """``num_categories`` when given, else ``floor(sqrt(n))`` kept inside ``[min_categories, max_categories]``;
        never more clusters than rows (reference :137-149)."""
        c = self.config
        if c.num_categories is not None:
            k = c.num_categories
        else:
            k = min(max(int(math.sqrt(max(n, 1))), c.min_categories), c.max_categories)
        return max(1, min(n, k))

    def _cluster(self, emb: np.ndarray, k: int) -> np.ndarray:
        c = self.config
        if c.cluster_algo.lower() != "kmeans":
            raise ValueError(f"Unsupported clustering algorithm '{c.cluster_algo}'. Only 'kmeans' is currently supported.")
        extra = {"random_state": c.seed, **c.kmeans_kwargs, **c.cluster_kwargs}
        try:
            from cuml.cluster import KMeans as GpuKMeans  # optional

            return np.asarray(GpuKMeans(n_clusters=k, **extra).fit_predict(emb))
        except ImportError:
            from sklearn.cluster import KMeans

            return KMeans(n_clusters=k, **{"n_init": 10, **extra}).fit_predict(emb)

    # -- entry point ----------------------------------------------------------------------------------
    def __call__(self, dataset) -> Dict[str, Any]:
        if isinstance(dataset, torch.utils.data.IterableDataset):
            raise NotImplementedError("Iterable (or streaming) datasets are not yet supported for auto categorization. "
                                      "Please use a non-iterable dataset.")
        if len(dataset) == 0:
            raise ValueError("Cannot auto-categorize an empty dataset")
        texts = self._texts(dataset)
        emb = self._embed(texts)
        k = self._num_clusters(len(texts))
        labels = self._cluster(emb, k)
        out: Dict[str, Any] = {}
        for cid in sorted(set(int(x) for x in labels)):
            idx = [i for i, l in enumerate(labels) if int(l) == cid]
            name = f"{self.config.category_prefix}_{cid}"
            out[name] = dataset.select(idx) if hasattr(dataset, "select") else [dataset[i] for i in idx]
        return out
