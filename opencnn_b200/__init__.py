"""opencnn_b200: B200-native (sm_100a) Winograd F(2x2,3x3) convolution, a drop-in for the
operator surface of UDC-GAC/openCNN.  The product is the CUDA library behind the C ABI in
include/opencnn_b200.h; this package is its loader and a thin host-side mirror of the
reference's interface."""
from .api import (HostPlan, call_like_reference, conv3x3, conv3x3_noalloc, convolutionForward, convolutionForward_32x64x8,
                  filter_transform, last_device_status, tiles_dim, variant_name, winograd_forward,
                  workspace_bytes)
from .build import VARIANTS, build_all, build_variant

__all__ = ["HostPlan", "call_like_reference", "conv3x3", "conv3x3_noalloc", "convolutionForward", "convolutionForward_32x64x8",
           "filter_transform", "last_device_status", "tiles_dim", "variant_name", "winograd_forward",
           "workspace_bytes", "VARIANTS", "build_all", "build_variant"]
