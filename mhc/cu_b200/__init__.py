"""B200-native kernels of the mHC layer hot path and the host-side mirror of the reference's
operator interface.  ``capi`` wraps the C ABI of libmhc_b200.so; ``ops`` / ``layer`` carry the
reference's Python API (``MHCLayer``, ``sinkhorn_knopp``, ``rmsnorm``, ``mhc_layer_fused*``)."""
