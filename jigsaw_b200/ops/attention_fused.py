"""Bindings of the fused kernels (see the package docstring)."""

from __future__ import annotations


def __getattr__(name: str):
    if name.startswith("maybe_fused_"):
        return lambda *a, **k: None
    raise AttributeError(name)
