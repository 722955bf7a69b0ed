"""ctypes binding of libluxlib_b200.so — the same symbols, argument order and layouts the Julia
`ccall` shim uses (see include/luxlib_b200.h). Fails loudly when the library is missing: there is
no CPU or vendor-library fallback behind these calls."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(os.path.dirname(_HERE), "lib", "libluxlib_b200.so")

OK, BAD_ARG, BAD_SHAPE, BAD_ALIGN, UNSUPPORTED_DTYPE, LAUNCH_FAIL, TIMEOUT, WORKSPACE_TOO_SMALL = 0, -1, -2, -3, -4, -5, -6, -7
F32, BF16 = 0, 1
ACT_IDENTITY, ACT_RELU, ACT_GELU_TANH, ACT_GELU_ERF, ACT_TANH, ACT_SIGMOID, ACT_SWISH = range(7)
FLAG_TF32_1X, FLAG_FORCE_SIMT, FLAG_CTA_PAIR, FLAG_NO_CTA_PAIR, FLAG_X_COPY_GIVEN = 1, 2, 4, 8, 16


def flag_reserve_sms(n: int) -> int:
    """LB2_FLAG_RESERVE_SMS(n): the persistent GEMM of the call leaves n SMs free for a kernel running beside it."""
    return (int(n) & 0x7F) << 16


class ConvDesc(C.Structure):
    """lb2_conv_desc"""
    _fields_ = [
        ("ndim", C.c_int32), ("in_", C.c_int32 * 3), ("k", C.c_int32 * 3), ("stride", C.c_int32 * 3),
        ("pad_lo", C.c_int32 * 3), ("pad_hi", C.c_int32 * 3), ("dilation", C.c_int32 * 3),
        ("groups", C.c_int32), ("flipkernel", C.c_int32), ("cin", C.c_int32), ("cout", C.c_int32), ("batch", C.c_int32),
    ]


class PoolDesc(C.Structure):
    """lb2_pool_desc"""
    _fields_ = [
        ("ndim", C.c_int32), ("in_", C.c_int32 * 3), ("k", C.c_int32 * 3), ("stride", C.c_int32 * 3),
        ("pad_lo", C.c_int32 * 3), ("pad_hi", C.c_int32 * 3), ("dilation", C.c_int32 * 3),
        ("channels", C.c_int32), ("batch", C.c_int32),
    ]


POOL_MAX, POOL_MEAN = 0, 1


class OptLeaf(C.Structure):
    """lb2_opt_leaf"""
    _fields_ = [("param", C.c_void_p), ("grad", C.c_void_p), ("state1", C.c_void_p), ("state2", C.c_void_p),
                ("master", C.c_void_p), ("n", C.c_int64)]


OPT_DESCENT, OPT_MOMENTUM, OPT_ADAM = 0, 1, 2

_p, _i64, _i32, _u32, _sz, _dbl = C.c_void_p, C.c_int64, C.c_int32, C.c_uint32, C.c_size_t, C.c_double
_fp = C.c_void_p  # float* passed as raw device pointers

# name -> (restype, argtypes); exactly the declarations of include/luxlib_b200.h
PROTOTYPES = {
    "lb2_version": (_i32, []),
    "lb2_status_string": (C.c_char_p, [_i32]),
    "lb2_last_error_string": (C.c_char_p, []),
    "lb2_poll_device_status": (_i32, [_p]),
    "lb2_selftest_bounded_wait": (_i32, [C.c_uint64, _p]),
    "lb2_act_fwd": (_i32, [_p, _p, _i64, _i32, _i32, _p]),
    "lb2_act_bwd": (_i32, [_p, _p, _p, _p, _i64, _i32, _i32, _p]),
    "lb2_bias_act_fwd": (_i32, [_p, _p, _p, _i64, _i64, _i64, _i32, _i32, _p]),
    "lb2_bias_act_bwd_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "lb2_bias_act_bwd": (_i32, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _i32, _i32, _p, _sz, _p]),
    "lb2_dense_fwd_workspace_bytes": (_sz, [_i64, _i64, _i64, _i32, _u32]),
    "lb2_dense_fwd": (_i32, [_p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _i32, _u32, _p, _sz, _p]),
    "lb2_dense_bwd_workspace_bytes": (_sz, [_i64, _i64, _i64, _i32, _i32, _u32]),
    "lb2_dense_bwd": (_i32, [_p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _i32, _i32, _u32, _p, _sz, _p]),
    "lb2_matmul_workspace_bytes": (_sz, [_i64, _i64, _i64, _i32, _u32]),
    "lb2_matmul": (_i32, [_p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _i32, _i32, _i32, _u32, _p, _sz, _p]),
    "lb2_conv_output_size": (_i32, [C.POINTER(ConvDesc), C.POINTER(C.c_int32)]),
    "lb2_conv_fwd_workspace_bytes": (_sz, [C.POINTER(ConvDesc), _i32]),
    "lb2_conv_fwd": (_i32, [_p, _p, _p, _p, _p, C.POINTER(ConvDesc), _i32, _i32, _u32, _p, _sz, _p]),
    "lb2_conv_bwd_workspace_bytes": (_sz, [C.POINTER(ConvDesc), _i32, _i32]),
    "lb2_conv_bwd": (_i32, [_p, _p, _p, _p, _p, _p, _p, _p, C.POINTER(ConvDesc), _i32, _i32, _u32, _p, _sz, _p]),
    "lb2_batchnorm_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "lb2_batchnorm_fwd_train": (_i32, [_p, _fp, _fp, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _dbl, _dbl, _i32, _i32, _p, _sz, _p]),
    "lb2_batchnorm_fwd_train_static": (_i32, [_p, _fp, _fp, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _dbl, _dbl, _i32, _i32, _p]),
    "lb2_batchnorm_fwd_infer": (_i32, [_p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _dbl, _i32, _i32, _p]),
    "lb2_batchnorm_bwd": (_i32, [_p, _p, _p, _p, _p, _p, _p, _fp, _fp, _i64, _i64, _i64, _i32, _i32, _p, _sz, _p]),
    "lb2_batchnorm_bwd_infer": (_i32, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i64, _dbl, _i32, _i32, _p, _sz, _p]),
    "lb2_groupnorm_fwd": (_i32, [_p, _fp, _fp, _p, _p, _p, _i64, _i64, _i64, _i64, _dbl, _i32, _i32, _p]),
    "lb2_groupnorm_bwd_workspace_bytes": (_sz, [_i64, _i64, _i64, _i64]),
    "lb2_groupnorm_bwd": (_i32, [_p, _p, _p, _p, _p, _p, _p, _fp, _fp, _i64, _i64, _i64, _i64, _i32, _i32, _p, _sz, _p]),
    "lb2_pool_output_size": (_i32, [C.POINTER(PoolDesc), C.POINTER(C.c_int32)]),
    "lb2_pool_fwd": (_i32, [_p, _p, C.POINTER(PoolDesc), _i32, _i32, _p]),
    "lb2_pool_bwd": (_i32, [_p, _p, _p, _p, C.POINTER(PoolDesc), _i32, _i32, _p]),
    "lb2_conv_fwd_leaves_x_copy": (_i32, [_p, _i32]),
    "lb2_last_gemm_plan": (_i32, [C.POINTER(C.c_int32), _i32]),
    "lb2_cross_entropy_workspace_bytes": (_sz, [_i64, _i64]),
    "lb2_cross_entropy": (_i32, [_fp, _p, _p, _p, _i64, _i64, _i32, C.c_double, C.c_double, _i32, _p, _sz, _p]),
    "lb2_batched_matmul_workspace_bytes": (_sz, [_i64, _i64, _i64, _i32, C.c_uint32]),
    "lb2_batched_matmul": (_i32, [_p, _p, _p, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i32, _i32, _i32, _i32,
                                  C.c_uint32, _p, _sz, _p]),
    "lb2_attention_softmax_fwd": (_i32, [_p, _p, _p, _i64, _p, _i64, _i32, C.c_double, _i64, _i64, _i64, _i32, _p]),
    "lb2_attention_softmax_bwd": (_i32, [_p, _p, _p, _p, C.c_double, _i64, _i64, _i64, _i32, _p]),
    "lb2_conv_fwd_sums_is_fused": (_i32, [_p, _i32]),
    "lb2_conv_fwd_sums_workspace_bytes": (_sz, [_p, _i32]),
    "lb2_conv_fwd_sums": (_i32, [_p, _fp, _p, _p, _p, _i32, C.c_uint32, _p, _sz, _p]),
    "lb2_channel_sums_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "lb2_channel_sums": (_i32, [_fp, _p, _i64, _i64, _i64, _i32, _p, _sz, _p]),
    "lb2_batchnorm_fwd_train_sums": (_i32, [_p, _fp, _fp, _p, _p, _p, _p, _p, _p, _p, _fp, _i64, _i64, _i64, _dbl, _dbl, _i32, _i32, _p, _sz, _p]),
    "lb2_scale_fwd": (_i32, [_p, _p, _p, _p, _i64, _i64, _i32, _i32, _p]),
    "lb2_scale_bwd_workspace_bytes": (_sz, [_i64, _i64]),
    "lb2_scale_bwd": (_i32, [_p, _p, _p, _p, _p, _p, _p, _i64, _i64, _i32, _i32, _p, _sz, _p]),
    "lb2_mse_loss_workspace_bytes": (_sz, [_i64]),
    "lb2_mse_loss": (_i32, [_fp, _p, _p, _p, _i64, _i32, _p, _sz, _p]),
    "lb2_optimizer_step": (_i32, [C.POINTER(OptLeaf), _i32, _i32, _dbl, _dbl, _dbl, _dbl, _i64, _dbl, _i32, _p]),
    "lb2_instancenorm_update_stats": (_i32, [_p, _p, _p, _p, _fp, _fp, _i64, _i64, _i64, _dbl, _dbl, _i32, _p]),
    "lb2_layernorm_fwd": (_i32, [_p, _fp, _fp, _p, _p, _p, _i64, _i64, _dbl, _i32, _i32, _p]),
    "lb2_layernorm_bwd_workspace_bytes": (_sz, [_i64, _i64]),
    "lb2_layernorm_bwd": (_i32, [_p, _p, _p, _p, _p, _p, _p, _fp, _fp, _i64, _i64, _i32, _i32, _p, _sz, _p]),
}


class LuxLibB200Error(RuntimeError):
    """A non-zero status from the library (the Julia shim throws the same way)."""

    def __init__(self, status: int, message: str):
        super().__init__(f"libluxlib_b200 status {status}: {message}")
        self.status = status


class DimensionMismatch(ValueError):
    """Julia's DimensionMismatch (lib/LuxLib/src/impl/matmul.jl:21-34)."""


class ArgumentError(ValueError):
    """Julia's ArgumentError (lib/LuxLib/src/api/groupnorm.jl:40-67)."""


_lib = None


def load():
    """Returns the loaded library; raises when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python lux.jl_b200/build.py` (nvcc, sm_100a). "
            "luxlib_b200 has no CPU or vendor-library fallback.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError when a declared symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status: int) -> None:
    if status == OK:
        return
    lib = load()
    msg = lib.lb2_last_error_string().decode() or lib.lb2_status_string(status).decode()
    if status == BAD_SHAPE:
        raise DimensionMismatch(msg)
    raise LuxLibB200Error(status, msg)
