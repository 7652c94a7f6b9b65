"""Utilities around the training loop: CUDA-graph capture of a whole step, device timers."""

from .graph import GraphedStep
from .timing import DeviceTimer, nvtx_range

__all__ = ["DeviceTimer", "GraphedStep", "nvtx_range"]
