"""CPU-only checks of the drop-in boundary: the shared library loads, exports every symbol that
include/luxlib_b200.h declares, and rejects bad arguments with the documented status codes before
anything is launched (so none of this needs a GPU)."""
import ctypes as C
import os
import re

import pytest

import luxlib_b200 as L
from luxlib_b200 import _cabi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "luxlib_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    return sorted(set(re.findall(r"LB2_API[^;(]*?\b(lb2_\w+)\s*\(", text)))


def test_header_declares_the_whole_path():
    names = declared_symbols()
    for needed in ["lb2_dense_fwd", "lb2_dense_bwd", "lb2_conv_fwd", "lb2_conv_bwd", "lb2_batchnorm_fwd_train",
                   "lb2_batchnorm_fwd_infer", "lb2_batchnorm_bwd", "lb2_groupnorm_fwd", "lb2_groupnorm_bwd",
                   "lb2_layernorm_fwd", "lb2_layernorm_bwd", "lb2_bias_act_fwd", "lb2_bias_act_bwd", "lb2_act_fwd",
                   "lb2_act_bwd", "lb2_matmul"]:
        assert needed in names


def test_library_exports_every_declared_symbol():
    lib = _cabi.load()
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
        assert name in _cabi.PROTOTYPES, f"{name} has no ctypes prototype"
    assert set(_cabi.PROTOTYPES) == set(declared_symbols())
    assert lib.lb2_version() >= 100


def test_every_declaration_cites_the_reference_or_says_it_has_no_counterpart():
    text = open(HEADER).read()
    # each exported compute entry point is preceded by a comment naming a LuxLib / Lux source file
    for name in declared_symbols():
        if name.endswith("_workspace_bytes") or name in ("lb2_version", "lb2_status_string"):
            continue
        idx = text.index(name + "(")
        window = text[max(0, idx - 1600):idx]
        assert re.search(r"(lib/LuxLib|src/layers|src/distributed|src/helpers|no counterpart in the reference)", window), name


def test_status_codes_for_bad_arguments():
    lib = _cabi.load()
    assert lib.lb2_bias_act_fwd(None, None, None, 4, 4, 4, 7, 0, None) == _cabi.UNSUPPORTED_DTYPE
    assert b"dtype" in lib.lb2_last_error_string()
    assert lib.lb2_bias_act_fwd(None, None, None, 4, 4, 4, _cabi.F32, 99, None) == _cabi.BAD_ARG
    assert lib.lb2_bias_act_fwd(None, None, None, 4, 4, 4, _cabi.F32, 0, None) == _cabi.BAD_ARG  # null pointers
    assert lib.lb2_bias_act_fwd(None, None, None, 0, 4, 4, _cabi.F32, 0, None) == _cabi.OK       # zero-sized
    assert lib.lb2_bias_act_fwd(1, 2, None, 4, 4, 4, _cabi.F32, 0, None) == _cabi.BAD_ALIGN
    assert lib.lb2_dense_fwd(None, None, None, None, None, 4, 4, 4, 2, 4, 4, 0, 0, 0, None, 0, None) == _cabi.BAD_SHAPE
    assert lib.lb2_dense_fwd(None, None, None, None, None, 0, 4, 4, 1, 4, 1, 0, 0, 0, None, 0, None) == _cabi.OK
    assert lib.lb2_groupnorm_fwd(None, None, None, None, None, None, 4, 6, 4, 2, 1e-5, 0, 0, None) == _cabi.BAD_SHAPE
    assert lib.lb2_layernorm_fwd(None, None, None, None, None, None, 0, 5, 1e-5, 0, 0, None) == _cabi.OK
    assert lib.lb2_batchnorm_fwd_infer(None, None, None, None, None, None, 1, 2, 3, 1e-5, 0, 0, None) == _cabi.BAD_ARG
    assert lib.lb2_act_bwd(16, 16, None, None, 8, 0, _cabi.ACT_GELU_TANH, None) == _cabi.BAD_ARG  # gelu needs pre
    assert lib.lb2_status_string(_cabi.TIMEOUT) == b"device-side wait timed out"


def test_status_codes_of_the_pooling_optimizer_and_instancenorm_entry_points():
    import ctypes as C
    lib = _cabi.load()
    d = _cabi.PoolDesc()
    d.ndim, d.channels, d.batch = 2, 3, 2
    for i in range(3):
        d.in_[i], d.k[i], d.stride[i], d.dilation[i] = (8, 2, 2, 1) if i < 2 else (1, 1, 1, 1)
    out = (C.c_int32 * 3)()
    assert lib.lb2_pool_output_size(C.byref(d), out) == _cabi.OK and (out[0], out[1]) == (4, 4)
    assert lib.lb2_pool_fwd(None, None, C.byref(d), _cabi.POOL_MAX, _cabi.F32, None) == _cabi.BAD_ARG      # null tensors
    assert lib.lb2_pool_fwd(None, None, C.byref(d), 7, _cabi.F32, None) == _cabi.BAD_ARG                   # unknown kind
    assert lib.lb2_pool_fwd(None, None, C.byref(d), _cabi.POOL_MAX, 9, None) == _cabi.UNSUPPORTED_DTYPE
    assert lib.lb2_pool_bwd(16, 16, None, None, C.byref(d), _cabi.POOL_MAX, _cabi.F32, None) == _cabi.BAD_ARG  # max needs y, x
    d.stride[0] = 0
    assert lib.lb2_pool_output_size(C.byref(d), out) == _cabi.BAD_SHAPE
    d.stride[0], d.batch = 2, 0
    assert lib.lb2_pool_fwd(None, None, C.byref(d), _cabi.POOL_MEAN, _cabi.F32, None) == _cabi.OK          # empty batch
    leaf = (_cabi.OptLeaf * 1)()
    leaf[0].param, leaf[0].grad, leaf[0].n = 16, 32, 4
    assert lib.lb2_optimizer_step(leaf, 1, 5, 0.1, 0.9, 0.999, 1e-8, 1, 1.0, _cabi.F32, None) == _cabi.BAD_ARG      # unknown rule
    assert lib.lb2_optimizer_step(leaf, 1, _cabi.OPT_ADAM, 0.1, 0.9, 0.999, 1e-8, 1, 1.0, _cabi.F32, None) == _cabi.BAD_ARG   # no state
    assert lib.lb2_optimizer_step(leaf, 1, _cabi.OPT_DESCENT, 0.1, 0.9, 0.999, 1e-8, 0, 1.0, _cabi.F32, None) == _cabi.BAD_ARG  # step from 1
    leaf[0].param = 18
    assert lib.lb2_optimizer_step(leaf, 1, _cabi.OPT_DESCENT, 0.1, 0.0, 0.0, 0.0, 1, 1.0, _cabi.F32, None) == _cabi.BAD_ALIGN
    assert lib.lb2_optimizer_step(None, 0, _cabi.OPT_DESCENT, 0.1, 0.0, 0.0, 0.0, 1, 1.0, _cabi.F32, None) == _cabi.OK         # nothing to do
    assert lib.lb2_instancenorm_update_stats(None, None, None, None, None, None, 4, 3, 2, 0.1, 1e-5, _cabi.F32, None) == _cabi.BAD_ARG
    assert lib.lb2_instancenorm_update_stats(None, None, None, None, None, None, 4, 0, 2, 0.1, 1e-5, _cabi.F32, None) == _cabi.OK


def test_static_scratch_entry_point_rejects_oversized_problems_before_touching_the_gpu():
    lib = _cabi.load()
    S, C, B = 1, 1 << 18, 2
    assert lib.lb2_batchnorm_workspace_bytes(S, C, B) > (4 << 20)
    rc = lib.lb2_batchnorm_fwd_train_static(16, 16, 16, None, None, 16, None, None, None, None, S, C, B, 0.1, 1e-5,
                                            _cabi.F32, _cabi.ACT_IDENTITY, None)
    assert rc == _cabi.WORKSPACE_TOO_SMALL and b"built-in scratch" in lib.lb2_last_error_string()


def test_conv_descriptor_and_output_size():
    lib = _cabi.load()
    d = _cabi.ConvDesc()
    d.ndim = 2
    for i, (n, k, s, lo, hi, dil) in enumerate([(28, 3, 1, 0, 1, 1), (28, 3, 1, 1, 2, 1)]):
        d.in_[i], d.k[i], d.stride[i], d.pad_lo[i], d.pad_hi[i], d.dilation[i] = n, k, s, lo, hi, dil
    d.groups, d.flipkernel, d.cin, d.cout, d.batch = 1, 0, 1, 1, 1
    out = (C.c_int32 * 3)()
    assert lib.lb2_conv_output_size(C.byref(d), out) == _cabi.OK
    assert (out[0], out[1]) == (27, 29)   # test/core_layers/conv_tests.jl:53-69
    d.groups = 2
    assert lib.lb2_conv_output_size(C.byref(d), out) == _cabi.BAD_SHAPE
    assert C.sizeof(_cabi.ConvDesc) == 4 * (1 + 18 + 5)


def test_workspace_queries_are_pure_functions_of_the_extents():
    lib = _cabi.load()
    assert lib.lb2_dense_fwd_workspace_bytes(4096, 8192, 4096, _cabi.BF16, 0) == 0
    f32 = lib.lb2_dense_fwd_workspace_bytes(256, 128, 784, _cabi.F32, 0)
    assert f32 == 2 * (256 * 784 * 4 + 784 * 128 * 4)
    assert lib.lb2_dense_fwd_workspace_bytes(256, 128, 784, _cabi.F32, _cabi.FLAG_TF32_1X) == 0
    assert lib.lb2_groupnorm_bwd_workspace_bytes(1024, 512, 32, 128) == 512 * 128 * 2 * 4
    assert lib.lb2_layernorm_bwd_workspace_bytes(0, 5) == 0


def test_host_mirror_argument_errors_need_no_gpu():
    import torch
    x = torch.zeros(4, 6)
    with pytest.raises(L.ArgumentError):
        L.ops._gn_sizes(torch.zeros(3, 3, 5, 2), 2)
    with pytest.raises(L.ArgumentError):
        L.ops._ln_rows(x, None, None, None)
    with pytest.raises(L.ArgumentError):
        L.ops.act_code("softplus")
    assert L.ops._ln_rows(torch.zeros(4, 4, 6, 3), torch.ones(4, 4, 6, 1), torch.ones(4, 4, 6, 1), (1, 2, 3)) == (96, 3)
    assert L.ops._ln_rows(torch.zeros(16, 7), torch.ones(16), torch.ones(16), None) == (16, 7)
    with pytest.raises(L.ArgumentError):  # dims=nothing with a rank-3 affine normalises dim 1 only: generic path
        L.ops._ln_rows(torch.zeros(4, 4, 6, 3), torch.ones(4, 4, 6), torch.ones(4, 4, 6), None)
    assert L.ops._scb(torch.zeros(5, 4, 3, 2)) == (20, 3, 2)
    assert L.needs_preactivation("gelu") and not L.needs_preactivation("tanh_fast")
    assert abs(L.default_epsilon(torch.float32) - 1.1337e-5) < 1e-8
    assert abs(L.default_epsilon(torch.bfloat16) - 0.03125) < 1e-9
    t = L.jl_empty((3, 4, 5), torch.float32, "cpu")
    assert t.stride() == (1, 3, 12) and L.is_colmajor(t)
    import numpy as np
    a = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    j = L.from_numpy(a, "cpu")
    assert L.is_colmajor(j) and (L.to_numpy(j) == a).all()


def test_the_library_reads_no_environment_variable():
    # a drop-in library must not change its arithmetic on an inherited environment: every switch is an argument
    import glob
    csrc = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lux.jl_b200", "csrc")
    files = sorted(glob.glob(os.path.join(csrc, "*.cu")) + glob.glob(os.path.join(csrc, "*.cuh")))
    assert files
    for f in files:
        with open(f) as fh:
            text = fh.read()
        assert "getenv" not in text, f
