"""luxlib_b200 — host-side mirror of LuxLib's fused-layer operator API over libluxlib_b200.so
(hand-written sm_100a kernels). Importing this package never touches a GPU; the first op call
loads the shared library and fails loudly if it has not been built."""
from . import _cabi
from ._cabi import ArgumentError, DimensionMismatch, LuxLibB200Error
from .arrays import as_colmajor, from_numpy, is_colmajor, jl_empty, jl_zeros, to_numpy
from .ops import (ConvDims, PoolDims, add_activation, batchnorm, bias_activation, default_epsilon, fast_activation,
                  fused_conv_bias_activation, fused_dense_bias_activation, groupnorm, instancenorm, layernorm, matmul, maxpool, meanpool,
                  needs_preactivation, rrule_add_activation, rrule_batchnorm, rrule_bias_activation, rrule_fused_conv,
                  rrule_fused_dense, rrule_groupnorm, rrule_instancenorm, rrule_layernorm, rrule_maxpool, rrule_meanpool, mse_loss,
                  rrule_mse_loss, conv_transpose_bias_activation, rrule_conv_transpose, conv_transpose_output_size, scale, rrule_scale, cross_entropy_loss, rrule_cross_entropy_loss, batched_matmul, rrule_batched_matmul,
                  scaled_dot_product_attention, rrule_scaled_dot_product_attention, rrule_conv_batchnorm)

__all__ = [
    "ArgumentError", "DimensionMismatch", "LuxLibB200Error", "ConvDims", "PoolDims",
    "as_colmajor", "from_numpy", "is_colmajor", "jl_empty", "jl_zeros", "to_numpy",
    "fused_dense_bias_activation", "fused_conv_bias_activation", "batchnorm", "groupnorm", "instancenorm", "layernorm",
    "bias_activation", "add_activation", "rrule_add_activation", "fast_activation", "matmul", "default_epsilon", "needs_preactivation",
    "rrule_fused_dense", "rrule_fused_conv", "rrule_batchnorm", "rrule_groupnorm", "rrule_instancenorm", "rrule_layernorm", "maxpool", "meanpool", "rrule_maxpool", "rrule_meanpool",
    "rrule_bias_activation", "mse_loss", "rrule_mse_loss", "conv_transpose_bias_activation", "rrule_conv_transpose", "conv_transpose_output_size", "scale", "rrule_scale", "cross_entropy_loss", "rrule_cross_entropy_loss", "batched_matmul", "rrule_batched_matmul",
    "scaled_dot_product_attention", "rrule_scaled_dot_product_attention", "rrule_conv_batchnorm",
]
