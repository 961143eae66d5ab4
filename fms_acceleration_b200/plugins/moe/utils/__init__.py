from .scattermoe_prepare import prepare_scattermoe  # noqa: F401
