"""B200-native LayerAdam path for SlideFormer-style layer-sliding fine-tuning.

The package holds the fused sm_100a optimizer kernel behind a C ABI (csrc/, include/) and the
host-side mirror of the reference's interfaces for that path.  Importing the package does not
load the native library; the first optimizer object does, and fails loudly if it is missing.
"""
from .layer_adam import LayerAdam  # noqa: F401

__all__ = ["LayerAdam"]
