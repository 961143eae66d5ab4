"""``torch_custom_op``: register a function that mutates some of its arguments as a ``torch.library`` custom
operator when this torch offers that, and hand it back unchanged otherwise (the reference's
scattermoe_utils/khd/custom_op.py:16-47, where the registration makes Triton launchers traceable).  Nothing in this
package is traced by a compiler, so registration is optional and off unless asked for."""
from __future__ import annotations

from typing import Callable, Iterable, Optional

import torch


class _IdentityOp:
    """What the decorator returns when nothing is registered: the function itself, with the ``register_fake`` hook
    of a real custom operator accepted and ignored."""

    def __init__(self, fn: Callable) -> None:
        self.fn = fn
        self.__name__ = getattr(fn, "__name__", "op")
        self.__doc__ = fn.__doc__

    def __call__(self, *args, **kwargs):
        return self.fn(*args, **kwargs)

    def register_fake(self, fn: Callable) -> Callable:
        return fn


def torch_custom_op(name: str, fn: Optional[Callable] = None, /, *, mutates_args: Iterable[str] | str = (),
                    device_types=None, schema: Optional[str] = None, register: bool = False):
    def wrap(f: Callable):
        if register and hasattr(torch, "library") and hasattr(torch.library, "custom_op"):
            return torch.library.custom_op(name, f, mutates_args=mutates_args, device_types=device_types, schema=schema)
        return _IdentityOp(f)

    return wrap if fn is None else wrap(fn)
