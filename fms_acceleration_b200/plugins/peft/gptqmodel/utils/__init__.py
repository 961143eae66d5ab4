from .backend import Backend  # noqa: F401
