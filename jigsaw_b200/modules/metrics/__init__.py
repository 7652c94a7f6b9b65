"""Distributed segmentation metrics."""

from ..._core.public import set_module
from ._segmentation import DistributedSegmentationMetrics, confusion_to_metrics, distributed_confusion_matrix

__all__ = ["DistributedSegmentationMetrics", "confusion_to_metrics", "distributed_confusion_matrix"]

set_module(globals(), __all__)
