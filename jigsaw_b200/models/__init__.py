"""Model families assembled from the distributed layers (benchmark configurations)."""

from .cnn import DomainCNN
from .swin import Swin, SwinConfig
from .unet3d import UNet3d, UNet3dConfig
from .vit import ViT, ViTConfig

__all__ = ["DomainCNN", "Swin", "SwinConfig", "UNet3d", "UNet3dConfig", "ViT", "ViTConfig"]
