"""Guard against passing a kernel configuration built for another layer.

Reference parity: jigsaw/_core/config.py:6-34.
"""

from __future__ import annotations

from typing import Any


def check_config(config: Any, expected: dict[str, Any]) -> None:
    """Raise ``ValueError`` if ``config._layer_key`` differs from the layer's ``expected`` properties."""
    key = getattr(config, "_layer_key", {})
    diff = [f"{k}={key.get(k)!r} (layer: {v!r})" for k, v in expected.items() if key.get(k) != v]
    if diff:
        raise ValueError("config was built for a different layer: " + ", ".join(diff) + ".")
