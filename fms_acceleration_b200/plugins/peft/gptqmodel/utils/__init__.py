from .backend import Backend  # noqa: F401
from .backend import get_backend  # noqa: F401,E402
