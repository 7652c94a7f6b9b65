"""Model families assembled from the distributed layers (benchmark configurations)."""

from .cnn import DomainCNN

__all__ = ["DomainCNN"]
