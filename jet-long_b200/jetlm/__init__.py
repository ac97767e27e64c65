"""jetlm — B200-native host package for the Jet-Long `jetlong_fused` attention path.

Import paths mirror the reference (`jetlm.kernels.cute_jetlong_backend`,
`jetlm.kernels.merge_fused`, `jetlm.modeling.jetlong_fused`) so its callers switch unchanged.
"""
__version__ = "0.1.0"
