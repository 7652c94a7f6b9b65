"""Label public objects with the module path they are documented under.

Reference parity: jigsaw/_core/public.py:7-33 (reprs and pickles name the public path).
"""

from __future__ import annotations

import inspect
from typing import Any


def set_module(namespace: dict[str, Any], names: list[str] | tuple[str, ...]) -> None:
    """Set ``__module__`` of every class / function in ``names`` to the package in ``namespace``."""
    public = namespace["__name__"]
    for name in names:
        obj = namespace.get(name)
        if obj is None or inspect.ismodule(obj):
            continue
        if inspect.isclass(obj) or inspect.isfunction(obj):
            try:
                obj.__module__ = public
            except (AttributeError, TypeError):
                pass
