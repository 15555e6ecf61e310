"""s2cnn_b200 - B200-native (sm_100a) implementation of the spectral hot path of s2cnn.

Drop-in for the reference's public names: ``from s2cnn import X`` becomes
``from s2cnn_b200 import X`` (the same sub-module paths exist too, e.g.
``s2cnn_b200.soft.so3_fft.so3_rfft``).  All ops run hand-written CUDA kernels through the C ABI in
``include/s2cnn_b200.h``; there is no CPU or eager fallback.
"""
from .s2_ft import s2_rft
from .so3_ft import so3_rft
from .s2_grid import s2_near_identity_grid, s2_equatorial_grid, s2_soft_grid
from .so3_grid import so3_near_identity_grid, so3_equatorial_grid, so3_soft_grid
from .s2_mm import s2_mm
from .so3_mm import so3_mm
from .soft import (S2Convolution, SO3Convolution, SO3Shortcut, so3_integrate, so3_relu_integrate,
                   so3_rotation)
from .fuse import fuse
from . import models, projection
from .tables import set_table_cache_dir

__all__ = [
    "s2_rft", "so3_rft", "s2_near_identity_grid", "s2_equatorial_grid", "s2_soft_grid",
    "so3_near_identity_grid", "so3_equatorial_grid", "so3_soft_grid", "s2_mm", "so3_mm",
    "so3_rotation",
    "S2Convolution", "SO3Convolution", "SO3Shortcut", "so3_integrate", "so3_relu_integrate",
    "fuse", "models", "projection", "set_table_cache_dir",
]
