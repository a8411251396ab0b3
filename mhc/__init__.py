"""Drop-in for the ``mhc`` package of AndreSlavescu/mHC.cu (src/python/mhc/__init__.py:1-15):
the same public names, running on hand-written sm_100a kernels (``mhc.cu_b200``)."""
from .cu_b200.layer import MHCBlock, MHCLayer
from .cu_b200.ops import (
    sinkhorn_knopp,
    rmsnorm,
    mhc_layer_fused,
    mhc_layer_fused_dynamic,
    mhc_layer_fused_inference,
    mhc_pre,
    mhc_post,
)

__all__ = [
    "MHCLayer",
    "sinkhorn_knopp",
    "rmsnorm",
    "mhc_layer_fused",
    "mhc_layer_fused_dynamic",
    # beyond the reference: the layer in two halves around a sub-layer
    "MHCBlock",
    "mhc_pre",
    "mhc_post",
]
