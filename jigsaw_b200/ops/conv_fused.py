"""Bindings of the halo-fused convolution kernels (filled in by the kernel layer)."""

from __future__ import annotations


def maybe_fused_conv2d(layer, x, w, b):
    return None
