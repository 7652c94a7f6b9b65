"""Segmentation metrics for predictions whose class axis, spatial axes or both are cut over ranks.

======================================  ==========================================================================
``distributed_confusion_matrix``        counts (target class, predicted class) pairs of the local tile and sums them
                                        over the groups that hold the other tiles; the arg-max over a cut class
                                        axis takes the lowest class index on a tie, as ``torch.argmax`` does
``confusion_to_metrics``                turns a confusion matrix into pixel accuracy, per-class and mean IoU, Dice,
                                        precision and recall (classes that never occur are left out of the means)
``DistributedSegmentationMetrics``      module that accumulates the matrix over batches (``update`` / ``compute`` /
                                        ``reset``), with ``ignore_index`` and excluded classes
======================================  ==========================================================================

Reference parity: jigsaw/modules/metrics/__init__.py (three public names).
"""

from ..._core.public import set_module
from ._segmentation import DistributedSegmentationMetrics, confusion_to_metrics, distributed_confusion_matrix

__all__ = ["DistributedSegmentationMetrics", "confusion_to_metrics", "distributed_confusion_matrix"]

set_module(globals(), __all__)
