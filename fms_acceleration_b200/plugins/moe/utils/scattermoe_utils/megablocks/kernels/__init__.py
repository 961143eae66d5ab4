from .gather_scatter import gather, padded_gather, padded_scatter, padded_scatter_wgrad, scatter, scatter_wgrad  # noqa: F401
