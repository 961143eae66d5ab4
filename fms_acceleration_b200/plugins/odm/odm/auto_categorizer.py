"""Pseudo-categories for a single un-labelled dataset: embed every sample, cluster with k-means, one category per
cluster (role of fms_acceleration_odm/odm/auto_categorizer.py:38-201).  The embedding model (sentence-transformers)
and cuML are optional; scikit-learn's KMeans is the default clusterer."""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import numpy as np


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
        self.config = config or AutoCategorizeConfig()

    # -- pieces ---------------------------------------------------------------------------------------
    def _texts(self, dataset) -> List[str]:
        c = self.config
        cols = getattr(dataset, "column_names", None)
        if cols is not None and c.input_column in cols:
            return [str(t) for t in dataset[c.input_column]]
        if c.tokenizer is not None:
            return [c.tokenizer.decode(dataset[i]["input_ids"], skip_special_tokens=True) for i in range(len(dataset))]
        raise ValueError(f"dataset has no column {c.input_column!r} and no tokenizer was given to rebuild the text")

    def _embed(self, texts: List[str]) -> np.ndarray:
        from sentence_transformers import SentenceTransformer  # optional dependency

        model = SentenceTransformer(self.config.model_name, **self.config.model_kwargs)
        emb = model.encode(texts, batch_size=self.config.batch_size, convert_to_numpy=True, normalize_embeddings=True,
                           show_progress_bar=False)
        return np.asarray(emb, dtype=np.float32)

    def _num_clusters(self, n: int) -> int:
        c = self.config
        k = c.num_categories if c.num_categories else int(round(math.sqrt(n)))
        return max(c.min_categories, min(c.max_categories, k, n))

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
