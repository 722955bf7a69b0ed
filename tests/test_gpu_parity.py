"""GPU parity tests: every op of the hot path, called through the C ABI (via the host mirror),
compared with the CPU oracle on identical seeded inputs.

Tolerances (the ones the path's contract states): fp32 outputs and gradients rel-L2 <= 1e-5;
bf16 storage with fp32 accumulation rel-L2 <= 1e-2; BatchNorm running statistics rel <= 1e-5.
"""
import numpy as np
import pytest
import torch

import luxlib_b200 as L
import parity_report
from oracle import luxlib_oracle as O

pytestmark = pytest.mark.gpu

TOL = {"f32": 1e-5, "bf16": 1e-2}
TDT = {"f32": torch.float32, "bf16": torch.bfloat16}
ACTS = ["identity", "relu", "gelu", "tanh", "sigmoid", "swish"]


def dev(a, dt):
    return None if a is None else L.from_numpy(a, "cuda", TDT[dt])


def prep(a, dt):
    """Oracle-side view of an input: bf16 rows see the bf16-rounded values."""
    if a is None:
        return None
    a = np.asarray(a, dtype=np.float32)
    return O.round_bf16(a) if dt == "bf16" else a


def check(got, want, dt, what, tol=None, scale=None, degenerate=False):
    """rel-L2 of got against want, asserted against the contract's tolerance and recorded in the parity report.

    The plain rel-L2 is what is asserted. Only a caller that states `degenerate=True` has the error judged against
    `scale` instead (an array naming the terms that cancel inside `want`): that is reserved for cases whose exact
    value is zero or nearly so by construction (BatchNorm statistics over 2 samples, a bias gradient behind a
    BatchNorm), where any fp32 evaluation, the reference's included, only returns rounding noise."""
    if want is None:
        assert got is None
        return
    g = L.to_numpy(got).astype(np.float64)
    w = np.asarray(want, dtype=np.float64)
    assert g.shape == w.shape, f"{what}: shape {g.shape} vs {w.shape}"
    assert np.isfinite(g).all(), f"{what}: non-finite values"
    limit = tol or TOL[dt]
    denom = np.linalg.norm(w.ravel())
    diff = np.linalg.norm((g - w).ravel())
    err = diff / denom if denom > 0 else np.linalg.norm(g.ravel())
    extra = {}
    if scale is not None:
        terms = np.linalg.norm(np.asarray(scale, dtype=np.float64).ravel())
        extra["cancellation"] = float(terms / denom) if denom > 0 else float("inf")
        if degenerate:
            extra["rel_l2_plain"] = float(err)
            err = diff / terms if terms > 0 else diff
            extra["judged"] = "against cancelling terms (degenerate case)"
    parity_report.record(what, dt, err, limit, **extra)
    assert err <= limit, f"{what}: rel-L2 {err:.3e} > {limit:.1e} {extra}"


# ------------------------------------------------------------------------------------------
# activation / bias-activation
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("act", ACTS)
@pytest.mark.parametrize("shape", [(5,), (7, 3), (4, 4, 6, 2), (8, 16, 3), (33, 5, 2), (1024, 8, 4)])
def test_bias_activation_fwd_bwd(dt, act, shape):
    rng = np.random.default_rng(10)
    x = prep(rng.standard_normal(shape), dt)
    c = shape[-2] if len(shape) > 1 else shape[0]
    b = prep(rng.uniform(-0.5, 0.5, c), dt)
    y_ref, pb_ref = O.bias_activation_rrule(act, x, b)
    y, pb = L.rrule_bias_activation(act, dev(x, dt), dev(b, dt))
    check(y, y_ref, dt, "y")
    delta = prep(rng.standard_normal(shape), dt)
    dx_ref, db_ref = pb_ref(delta)
    dx, db = pb(dev(delta, dt))
    check(dx, dx_ref, dt, "dx")
    check(db, db_ref, dt, "db")
    # no-bias variant == fast_activation
    check(L.fast_activation(act, dev(x, dt)), O.act_fn(act, x), dt, "fast_activation")


def test_zero_sized_arrays():
    # lib/LuxLib/test/common_ops/bias_act_tests.jl:119-131
    x = L.jl_empty((4, 3, 2, 0), torch.float32, "cuda")
    b = torch.zeros(2, device="cuda")
    assert L.bias_activation("relu", x, b).shape == (4, 3, 2, 0)
    assert L.fused_dense_bias_activation("relu", L.jl_empty((3, 0), torch.float32, "cuda"),
                                         L.jl_empty((0, 2), torch.float32, "cuda"), None).shape == (3, 2)


# ------------------------------------------------------------------------------------------
# dense
# ------------------------------------------------------------------------------------------
DENSE_SHAPES = [
    (4, 3, 4), (32, 3, 32), (10, 128, 256), (256, 128, 784),   # small / config-1 layers (CUDA cores or 3xTF32)
    (128, 256, 64), (256, 512, 512), (384, 200, 136), (130, 300, 72),  # tensor-core path incl. ragged tiles
]


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("act", ["identity", "relu", "gelu", "tanh", "swish"])
@pytest.mark.parametrize("mnk", DENSE_SHAPES)
def test_fused_dense_fwd_bwd(dt, act, mnk):
    M, N, K = mnk
    rng = np.random.default_rng(M * 7 + N * 3 + K)
    W = prep(O.glorot_uniform(rng, (M, K)), dt)
    x = prep(rng.standard_normal((K, N)), dt)
    b = prep(rng.uniform(-0.1, 0.1, M), dt)
    y_ref, pb_ref = O.fused_dense_rrule(act, W, x, b)
    y, pb = L.rrule_fused_dense(act, dev(W, dt), dev(x, dt), dev(b, dt))
    check(y, y_ref, dt, "y")
    delta = prep(rng.standard_normal((M, N)), dt)
    dW_ref, dx_ref, db_ref = pb_ref(delta)
    dW, dx, db = pb(dev(delta, dt))
    check(dW, dW_ref, dt, "dW")
    check(dx, dx_ref, dt, "dx")
    check(db, db_ref, dt, "db")
    assert L._cabi.load().lb2_poll_device_status(None) == 0


@pytest.mark.parametrize("dt", ["f32", "bf16"])
def test_dense_no_bias_and_vector_input(dt):
    rng = np.random.default_rng(11)
    W = prep(rng.standard_normal((24, 40)), dt)
    x = prep(rng.standard_normal(40), dt)
    y = L.fused_dense_bias_activation("sigmoid", dev(W, dt), dev(x, dt), None)
    check(y, O.act_fn("sigmoid", W @ x), dt, "y(vector)")
    with pytest.raises(L.DimensionMismatch):
        L.fused_dense_bias_activation("relu", dev(W, dt), dev(rng.standard_normal((39, 2)), dt), None)


def test_dense_known_answers():
    # test/core_layers/basic_tests.jl:151-193
    W = torch.ones(2, 10, device="cuda").T.contiguous().T
    x = L.from_numpy(np.concatenate([np.ones((10, 1)), 2 * np.ones((10, 1))], 1).astype(np.float32))
    y = L.fused_dense_bias_activation("identity", L.as_colmajor(W), x, torch.zeros(2, device="cuda"))
    assert (L.to_numpy(y) == np.array([[10, 20], [10, 20]])).all()


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("ta,tb", [(False, False), (True, False), (False, True), (True, True)])
def test_matmul_all_layouts(dt, ta, tb):
    rng = np.random.default_rng(12)
    M, N, K = 192, 264, 160
    A = prep(rng.standard_normal((K, M) if ta else (M, K)), dt)
    B = prep(rng.standard_normal((N, K) if tb else (K, N)), dt)
    ref = (A.T if ta else A) @ (B.T if tb else B)
    check(L.matmul(dev(A, dt), dev(B, dt), transA=ta, transB=tb), ref, dt, "C")


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("flags", [0, 4])  # single-CTA kernel (default) and CTA-pair kernel (LB2_FLAG_CTA_PAIR)
@pytest.mark.parametrize("mnk", [(2048, 2560, 512), (2100, 2330, 200), (2560, 2304, 2560), (2500, 2190, 2328)])
def test_fused_dense_large_tiles_both_tensor_core_kernels(dt, flags, mnk):
    M, N, K = mnk
    rng = np.random.default_rng(21)
    W = prep(O.glorot_uniform(rng, (M, K)), dt)
    x = prep(rng.standard_normal((K, N)), dt)
    b = prep(rng.uniform(-0.1, 0.1, M), dt)
    y_ref, pb_ref = O.fused_dense_rrule("gelu", W, x, b)
    y, pb = L.rrule_fused_dense("gelu", dev(W, dt), dev(x, dt), dev(b, dt), flags=flags)
    check(y, y_ref, dt, "y")
    delta = prep(rng.standard_normal((M, N)), dt)
    dW_ref, dx_ref, db_ref = pb_ref(delta)
    dW, dx, db = pb(dev(delta, dt))
    check(dW, dW_ref, dt, "dW")
    check(dx, dx_ref, dt, "dx")
    check(db, db_ref, dt, "db")
    assert L._cabi.load().lb2_poll_device_status(None) == 0


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("ta,tb", [(False, False), (True, False), (False, True), (True, True)])
def test_matmul_all_layouts_cta_pair_kernel(dt, ta, tb):
    rng = np.random.default_rng(22)
    M, N, K = 2304, 2250, 328
    A = prep(rng.standard_normal((K, M) if ta else (M, K)), dt)
    B = prep(rng.standard_normal((N, K) if tb else (K, N)), dt)
    ref = (A.T if ta else A) @ (B.T if tb else B)
    check(L.matmul(dev(A, dt), dev(B, dt), transA=ta, transB=tb, flags=L._cabi.FLAG_CTA_PAIR), ref, dt, "C")
    assert L._cabi.load().lb2_poll_device_status(None) == 0


def test_dense_tf32_single_pass_flag_is_looser_but_close():
    rng = np.random.default_rng(13)
    W, x = rng.standard_normal((256, 512)).astype(np.float32), rng.standard_normal((512, 256)).astype(np.float32)
    y = L.fused_dense_bias_activation("identity", dev(W, "f32"), dev(x, "f32"), None, flags=L._cabi.FLAG_TF32_1X)
    assert O.rel_l2(L.to_numpy(y), W @ x) < 2e-3
    y3 = L.fused_dense_bias_activation("identity", dev(W, "f32"), dev(x, "f32"), None)
    assert O.rel_l2(L.to_numpy(y3), W.astype(np.float64) @ x.astype(np.float64)) < 1e-5


ACCUMULATE_CASES = [
    # (M, N, K), flags: CUDA-core route (tiny), tensor-core single-CTA route with ragged tiles, forced CUDA-core
    # route, single-pass tf32, CTA-pair route (needs enough 256 x 256 tiles in all three GEMMs)
    ((20, 33, 17), 0), ((130, 300, 72), 0), ((256, 512, 512), 0), ((256, 512, 512), 2), ((256, 512, 512), 1),
    ((1792, 1800, 1792), 4),
]


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("act", ["identity", "relu", "gelu"])
@pytest.mark.parametrize("mnk,flags", ACCUMULATE_CASES)
def test_dense_pullback_accumulates_into_shadows(dt, act, mnk, flags):
    # Enzyme's reverse rule for fused_dense! (lib/LuxLib/src/impl/dense.jl:253-283): dW, dx and db are ADDED to the
    # shadows that already hold other contributions, and the output shadow is zeroed afterwards
    M, N, K = mnk
    if flags == 1 and dt == "bf16":
        pytest.skip("the single-pass tf32 flag only concerns Float32 storage")
    if flags == 1 and act == "relu":
        pytest.skip("a single-pass tf32 forward flips relu's mask where the pre-activation is within 1e-3 of zero")
    rng = np.random.default_rng(M + N + K + flags)
    W = prep(O.glorot_uniform(rng, (M, K)), dt)
    x = prep(rng.standard_normal((K, N)), dt)
    b = prep(rng.uniform(-0.1, 0.1, M), dt)
    delta = prep(rng.standard_normal((M, N)), dt)
    old = [prep(rng.standard_normal(shp) * s, dt) for shp, s in (((M, K), 3.0), ((K, N), 2.0), ((M,), 5.0))]
    _, pb_ref = O.fused_dense_rrule(act, W, x, b)
    grads = pb_ref(delta)
    y, pb = L.rrule_fused_dense(act, dev(W, dt), dev(x, dt), dev(b, dt), flags=flags)
    shadows = tuple(dev(o, dt) for o in old)
    d = dev(delta, dt)
    dW, dx, db = pb(d, shadows=shadows)
    assert dW.data_ptr() == shadows[0].data_ptr() and dx.data_ptr() == shadows[1].data_ptr()
    tol = 2e-3 if flags == 1 else None
    for name, got, o, g in zip(("dW", "dx", "db"), (dW, dx, db), old, grads):
        check(got, o.astype(np.float64) + np.asarray(g, np.float64), dt, f"{name} (accumulated)", tol=tol)
    assert float(d.abs().max()) == 0.0          # the output shadow is zeroed
    # a second pass adds once more
    d2 = dev(delta, dt)
    pb(d2, shadows=shadows)
    for name, got, o, g in zip(("dW", "dx", "db"), shadows, old, grads):
        check(got, o.astype(np.float64) + 2 * np.asarray(g, np.float64), dt, f"{name} (accumulated twice)", tol=tol)
    assert L._cabi.load().lb2_poll_device_status(None) == 0


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("ta", [False, True])
@pytest.mark.parametrize("tb", [False, True])
@pytest.mark.parametrize("mnk,flags", [((192, 264, 160), 0), ((9, 5, 30), 0), ((2304, 2250, 328), 4)])
def test_matmul_accumulates_into_a_strided_destination(dt, ta, tb, mnk, flags):
    # mul!(C, A, B, true, true) (lib/LuxLib/src/impl/matmul.jl:254-347) with C a column block view of a taller
    # matrix: the rows below the block must stay untouched
    M, N, K = mnk
    rng = np.random.default_rng(23)
    A = prep(rng.standard_normal((K, M) if ta else (M, K)), dt)
    B = prep(rng.standard_normal((N, K) if tb else (K, N)), dt)
    big = prep(rng.standard_normal((M + 8, N)), dt)
    ref = big.astype(np.float64).copy()
    ref[:M] += (A.T if ta else A).astype(np.float64) @ (B.T if tb else B).astype(np.float64)
    Cbig = dev(big, dt)
    out = L.matmul(dev(A, dt), dev(B, dt), transA=ta, transB=tb, flags=flags, out=Cbig[:M], accumulate=True)
    assert out.data_ptr() == Cbig.data_ptr()
    check(Cbig, ref, dt, "C (accumulated, ld > M)")
    assert L._cabi.load().lb2_poll_device_status(None) == 0


# ------------------------------------------------------------------------------------------
# convolution
# ------------------------------------------------------------------------------------------
CONV_CASES = [
    # spatial, k, cin, cout, stride, pad, dilation, groups, flip
    ((4, 4), (3, 3), 4, 8, 1, 0, 1, 1, False),
    ((4, 4), (3, 3), 4, 8, 1, 0, 1, 2, False),
    ((5, 4), (3, 3), 4, 8, 2, (1, 1), 1, 1, False),
    ((6, 5), (3, 2), 2, 4, (2, 1), (0, 1, 1, 2), 1, 1, True),
    ((9,), (3,), 2, 4, 1, 1, 2, 1, False),
    ((4, 4, 3), (2, 2, 2), 2, 2, 1, 0, 1, 1, False),
    ((16, 8), (3, 3), 16, 16, 1, 1, 1, 1, False),
]


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("act", ["identity", "sigmoid", "gelu"])
@pytest.mark.parametrize("case", CONV_CASES)
def test_fused_conv_fwd_bwd(dt, act, case):
    sp, k, cin, cout, stride, pad, dil, groups, flip = case
    nd = len(sp)
    rng = np.random.default_rng(14)
    x = prep(rng.standard_normal(sp + (cin, 2)), dt)
    w = prep(O.kaiming_normal(rng, k + (cin // groups, cout)), dt)
    b = prep(rng.uniform(-0.1, 0.1, cout), dt)
    ocd = O.ConvDims.make(nd, stride, pad, dil, groups, flip)
    lcd = L.ConvDims.make(nd, stride, pad, dil, groups, flip)
    y_ref, pb_ref = O.fused_conv_rrule(act, w, x, b, ocd)
    y, pb = L.rrule_fused_conv(act, dev(w, dt), dev(x, dt), dev(b, dt), lcd)
    check(y, y_ref, dt, "y")
    delta = prep(rng.standard_normal(y_ref.shape), dt)
    dw_ref, dx_ref, db_ref = pb_ref(delta)
    dw, dx, db = pb(dev(delta, dt))
    check(dw, dw_ref, dt, "dw")
    check(dx, dx_ref, dt, "dx")
    check(db, db_ref, dt, "db")


GENERAL_CONV_CASES = [
    # spatial, k, cin, cout, stride, pad, dilation, flip, batch — the geometries of a ResNet-18 beyond its stride-1
    # 64-channel stage, plus odd ones; bf16 storage takes the general tensor-core path (channel-innermost copies)
    ((32, 32), (7, 7), 3, 64, 2, 3, 1, False, 3),              # stem: kW taps folded into the channel index
    ((28, 28), (3, 3), 64, 128, 2, 1, 1, False, 3),            # strided 3x3 at a stage entry
    ((28, 28), (1, 1), 64, 128, 2, 0, 1, False, 3),            # 1x1 stride-2 projection (dx has untouched classes)
    ((14, 14), (3, 3), 128, 128, 1, 1, 1, False, 3),
    ((14, 14), (3, 3), 128, 256, 2, 1, 1, False, 2),
    ((7, 7), (3, 3), 256, 512, 1, 1, 1, False, 5),             # several images per tile, 256-wide N tiles
    ((7, 7), (3, 3), 512, 512, 1, 1, 1, True, 2),
    ((16, 12), (3, 3), 32, 48, 1, 2, 2, False, 2),             # dilation
    ((17, 13), (3, 2), 40, 24, (3, 2), (1, 0, 2, 1), 1, True, 2),   # odd strides, asymmetric padding
    ((150, 6), (3, 3), 16, 16, 1, 1, 1, False, 2),             # rows longer than a tile
    ((9, 9), (5, 5), 8, 8, 2, 2, 1, False, 2),
]


@pytest.mark.parametrize("act", ["identity", "relu", "gelu"])
@pytest.mark.parametrize("dt", ["bf16", "f32"])
@pytest.mark.parametrize("case", GENERAL_CONV_CASES)
def test_fused_conv_general_geometries(case, dt, act):
    sp, k, cin, cout, stride, pad, dil, flip, batch = case
    if dt == "f32" and act != "relu":
        pytest.skip("Float32 storage takes the direct kernels here; one activation is enough")
    rng = np.random.default_rng(29)
    x = prep(rng.standard_normal(sp + (cin, batch)), dt)
    w = prep(O.kaiming_normal(rng, k + (cin, cout)), dt)
    b = prep(rng.uniform(-0.1, 0.1, cout), dt)
    ocd = O.ConvDims.make(2, stride, pad, dil, 1, flip)
    lcd = L.ConvDims.make(2, stride, pad, dil, 1, flip)
    y_ref, pb_ref = O.fused_conv_rrule(act, w, x, b, ocd)
    y, pb = L.rrule_fused_conv(act, dev(w, dt), dev(x, dt), dev(b, dt), lcd)
    check(y, y_ref, dt, "y")
    delta = prep(rng.standard_normal(y_ref.shape), dt)
    dw_ref, dx_ref, db_ref = pb_ref(delta)
    dw, dx, db = pb(dev(delta, dt))
    check(dw, dw_ref, dt, "dw")
    check(dx, dx_ref, dt, "dx")
    check(db, db_ref, dt, "db")
    assert L._cabi.load().lb2_poll_device_status(None) == 0


TC_CONV_CASES = [
    # spatial, k, cin, cout, pad, flip  — shapes the tensor-core implicit-GEMM path takes (bf16, stride 1, W % 8 == 0)
    ((16, 8), (3, 3), 16, 16, 1, False),
    ((56, 12), (3, 3), 64, 64, 1, False),
    ((24, 9), (3, 3), 80, 72, (1, 1, 0, 2), True),
    ((32, 10), (1, 1), 64, 128, 0, False),
    ((40, 7), (5, 3), 32, 40, (2, 2, 1, 1), False),
    ((16, 6), (3, 3), 64, 96, 1, False),
    ((8, 40), (3, 5), 130, 48, (1, 1, 2, 2), False),
    ((12, 9), (3, 3), 24, 20, 1, False),     # W % 4 == 0 only: Float32 tensor-core path, bf16 direct path
    # at most 64 output channels: the bf16 filter gradient stacks kernel rows along M and cuts the taps out of the
    # unshifted tile in shared memory; one case per (kernel width, left padding) kind, odd and even kernel heights,
    # a row of a single 16-byte chunk, fewer than 64 positions, two channel chunks
    ((8, 5), (2, 2), 16, 24, (0, 1, 0, 1), False),
    ((24, 6), (2, 3), 32, 64, (1, 0, 1, 1), True),
    ((16, 7), (3, 1), 64, 48, (0, 2, 0, 0), False),
    ((16, 5), (3, 2), 24, 32, (2, 0, 1, 0), False),
    ((16, 6), (2, 4), 24, 32, (1, 0, 2, 1), False),
    ((32, 4), (4, 2), 40, 56, (1, 2, 0, 1), False),
    ((16, 6), (4, 2), 16, 16, (3, 0, 1, 0), True),
    ((16, 9), (1, 3), 128, 64, (0, 0, 1, 1), False),
    ((8, 3), (3, 3), 8, 8, 1, False),
    # output shorter / taller than the input: the bias gradient rides on the filter-gradient kernel only in the first
    ((16, 8), (3, 3), 16, 32, (1, 1, 0, 0), False),
    ((16, 4), (3, 3), 16, 32, (1, 1, 2, 2), False),
]


@pytest.mark.parametrize("force_simt", [False, True])
@pytest.mark.parametrize("act", ["identity", "relu", "gelu"])
@pytest.mark.parametrize("dt", ["bf16", "f32"])
@pytest.mark.parametrize("case", TC_CONV_CASES)
def test_fused_conv_tensor_core_path(case, dt, act, force_simt):
    sp, k, cin, cout, pad, flip = case
    rng = np.random.default_rng(23)
    x = prep(rng.standard_normal(sp + (cin, 3)), dt)
    w = prep(O.kaiming_normal(rng, k + (cin, cout)), dt)
    b = prep(rng.uniform(-0.1, 0.1, cout), dt)
    ocd = O.ConvDims.make(2, 1, pad, 1, 1, flip)
    lcd = L.ConvDims.make(2, 1, pad, 1, 1, flip)
    flags = L._cabi.FLAG_FORCE_SIMT if force_simt else 0
    y_ref, pb_ref = O.fused_conv_rrule(act, w, x, b, ocd)
    y, pb = L.rrule_fused_conv(act, dev(w, dt), dev(x, dt), dev(b, dt), lcd, flags=flags)
    check(y, y_ref, dt, "y")
    delta = prep(rng.standard_normal(y_ref.shape), dt)
    dw_ref, dx_ref, db_ref = pb_ref(delta)
    dw, dx, db = pb(dev(delta, dt))
    check(dw, dw_ref, dt, "dw")
    check(dx, dx_ref, dt, "dx")
    check(db, db_ref, dt, "db")
    assert L._cabi.load().lb2_poll_device_status(None) == 0


def test_conv_known_answers():
    # test/core_layers/conv_tests.jl:53-69 and :145-158
    x = L.from_numpy(np.ones((28, 28, 1, 1), np.float32))
    w = L.from_numpy(np.ones((3, 3, 1, 1), np.float32))
    y = L.to_numpy(L.fused_conv_bias_activation("relu", w, x, torch.zeros(1, device="cuda"),
                                                L.ConvDims.make(2, padding=(0, 1, 1, 2))))[:, :, 0, 0]
    assert y.shape == (27, 29)
    assert (y[0, 0], y[1, 1], y[-1, 0], y[0, -1], y[0, -2], y[-1, -1]) == (6, 9, 4, 3, 6, 2)
    img = np.zeros((7, 7, 1, 1), np.float32)
    img[3, 3] = 1
    wt = np.random.default_rng(0).standard_normal((3, 3, 1, 1)).astype(np.float32)
    y = L.to_numpy(L.fused_conv_bias_activation("identity", L.from_numpy(wt), L.from_numpy(img), None, L.ConvDims.make(2)))
    np.testing.assert_allclose(y[1:-1, 1:-1, 0, 0], wt[:, :, 0, 0], atol=1e-6)


# ------------------------------------------------------------------------------------------
# batchnorm
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("act", ["identity", "relu", "sigmoid"])
@pytest.mark.parametrize("shape", [(4, 4, 6, 2), (8, 2), (64, 48), (12, 12, 16, 8), (7, 5, 3, 4),
                                   # planes of 392 / 98 bytes: reductions four planes per round (8-byte / 2-byte loads), apply pass
                                   # in 16-byte vectors across plane boundaries; batch sizes that leave partial rounds
                                   (14, 14, 16, 4), (7, 7, 32, 6), (7, 7, 8, 41), (14, 14, 24, 37)])
@pytest.mark.parametrize("affine", [True, False])
def test_batchnorm_train_fwd_bwd(dt, act, shape, affine):
    _batchnorm_case(dt, act, shape, affine)


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("act", ["identity", "relu"])
@pytest.mark.parametrize("shape", [(96, 96, 40, 24), (256, 256, 4, 64)])
def test_batchnorm_large_tensors_take_the_single_launch_path(dt, act, shape):
    # above 16 MB the statistics and the normalisation run in one cooperative launch, one L2-sized group of
    # channels at a time; these shapes give one and several groups in either direction
    _batchnorm_case(dt, act, shape, True)
    assert L._cabi.load().lb2_poll_device_status(None) == 0


def _batchnorm_case(dt, act, shape, affine):
    rng = np.random.default_rng(15)
    c = shape[-2]
    x = prep(rng.standard_normal(shape) * rng.uniform(0.5, 2, (c, 1)) + 0.3, dt)
    g = prep(rng.uniform(0.5, 1.5, c), dt) if affine else None
    b = prep(rng.standard_normal(c) * 0.1, dt) if affine else None
    rm, rv = prep(rng.standard_normal(c) * 0.1, dt), prep(rng.uniform(0.5, 1.5, c), dt)
    z_ref, (rm_ref, rv_ref), pb_ref = O.batchnorm_rrule(x, g, b, rm, rv, True, act, 0.1, 1e-5)
    z, (nrm, nrv), pb = L.rrule_batchnorm(dev(x, dt), dev(g, dt), dev(b, dt), dev(rm, dt), dev(rv, dt), True, act, 0.1, 1e-5)
    check(z, z_ref, dt, "y")
    check(nrm, rm_ref, dt, "running_mean", tol=1e-5 if dt == "f32" else None)
    check(nrv, rv_ref, dt, "running_var", tol=1e-5 if dt == "f32" else None)
    delta = prep(rng.standard_normal(shape), dt)
    dx_ref, dg_ref, db_ref = pb_ref(delta)
    dx, dg, db = pb(dev(delta, dt))
    # dx = g' * (d - mean(d) - xhat * mean(d * xhat)) cancels; it is measured against the size of its terms
    x3 = x.reshape((-1,) + x.shape[-2:], order="F")
    inv = 1.0 / np.sqrt(x3.var(axis=(0, 2)) + 1e-5)
    gp = (inv if g is None else g * inv).reshape((1,) * (x.ndim - 2) + (c, 1))
    # statistics over at most 4 elements (the reference's (8, 2) test shape: 2 samples per channel) make dx vanish
    # analytically; only there is it judged on the size of its terms
    check(dx, dx_ref, dt, "dx", scale=delta * gp, degenerate=x3.shape[0] * x3.shape[2] <= 4)
    check(dg, dg_ref, dt, "dgamma")
    check(db, db_ref, dt, "dbeta")


def test_batchnorm_known_answers_and_modes():
    # test/core_layers/normalize_tests.jl:10-49
    x = L.from_numpy(np.array([[1, 3, 5], [2, 4, 6]], np.float32))
    one, zero = torch.ones(2, device="cuda"), torch.zeros(2, device="cuda")
    y, (rm, rv) = L.batchnorm(x, one, zero, zero.clone(), one.clone(), True, "identity", 0.1, 1e-5)
    np.testing.assert_allclose(L.to_numpy(y), [[-1.22474, 0, 1.22474]] * 2, atol=1e-5)
    np.testing.assert_allclose(L.to_numpy(rm), [0.3, 0.4], rtol=1e-6)
    np.testing.assert_allclose(L.to_numpy(rv), [1.3, 1.3], rtol=1e-6)
    yt, (rm2, rv2) = L.batchnorm(x, one, zero, rm, rv, False, "identity", 0.1, 1e-5)
    assert abs(L.to_numpy(yt)[0, 0] - (1 - 0.3) / np.sqrt(1.3)) < 1e-5
    assert rm2 is rm and rv2 is rv
    # training without running statistics: batch statistics, nothing returned
    y3, (a, b) = L.batchnorm(x, one, zero, None, None, True, "identity", 0.1, 1e-5)
    assert a is None and b is None
    np.testing.assert_allclose(L.to_numpy(y3), L.to_numpy(y), atol=1e-6)


@pytest.mark.parametrize("dt", ["f32", "bf16"])
def test_batchnorm_inference(dt):
    rng = np.random.default_rng(16)
    x = prep(rng.standard_normal((6, 5, 8, 3)), dt)
    g, b = prep(rng.uniform(0.5, 1.5, 8), dt), prep(rng.standard_normal(8), dt)
    rm, rv = prep(rng.standard_normal(8) * 0.2, dt), prep(rng.uniform(0.5, 2, 8), dt)
    y_ref, _ = O.batchnorm(x, g, b, rm, rv, False, "relu", 0.1, 1e-5)
    y, _ = L.batchnorm(dev(x, dt), dev(g, dt), dev(b, dt), dev(rm, dt), dev(rv, dt), False, "relu", 0.1, 1e-5)
    check(y, y_ref, dt, "y")


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("act", ["identity", "relu", "gelu"])
@pytest.mark.parametrize("shape", [(6, 5, 8, 3), (32, 40), (14, 14, 24, 16)])
@pytest.mark.parametrize("affine", [True, False])
def test_batchnorm_pullback_with_given_statistics(dt, act, shape, affine):
    # frozen BatchNorm (training = false, running statistics given): the reference's rrule
    # (lib/LuxLib/src/impl/batchnorm.jl:405-443) differentiates the affine-normalise step for the statistics it is handed
    rng = np.random.default_rng(19)
    c = shape[-2]
    x = prep(rng.standard_normal(shape) * 1.4 + 0.3, dt)
    g = prep(rng.uniform(0.5, 1.5, c), dt) if affine else None
    b = prep(rng.standard_normal(c) * 0.1, dt) if affine else None
    rm, rv = prep(rng.standard_normal(c) * 0.2, dt), prep(rng.uniform(0.5, 2, c), dt)
    z_ref, _, pb_ref = O.batchnorm_rrule(x, g, b, rm, rv, False, act, 0.1, 1e-5)
    z, (srm, srv), pb = L.rrule_batchnorm(dev(x, dt), dev(g, dt), dev(b, dt), dev(rm, dt), dev(rv, dt), False, act, 0.1, 1e-5)
    check(z, z_ref, dt, "y")
    check(srm, rm, dt, "running_mean unchanged")
    delta = prep(rng.standard_normal(shape), dt)
    dx_ref, dg_ref, db_ref = pb_ref(delta)
    dx, dg, db = pb(dev(delta, dt))
    check(dx, dx_ref, dt, "dx")
    check(dg, dg_ref, dt, "dgamma")
    check(db, db_ref, dt, "dbeta")


# ------------------------------------------------------------------------------------------
# groupnorm / layernorm
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("act", ["identity", "relu", "gelu"])
@pytest.mark.parametrize("shape,groups", [((6, 2), 2), ((4, 4, 6, 2), 3), ((2, 2, 6, 2), 2), ((16, 16, 32, 4), 4),
                                          ((32, 32, 16, 3), 2), ((8, 128, 64, 2), 4), ((7, 3, 10, 2), 5),
                                          # rows streamed in chunks: ragged last chunk, forward-only eligibility,
                                          # more rows than resident CTAs
                                          ((16, 16, 80, 2), 2), ((6, 6, 256, 2), 2), ((32, 32, 32, 40), 8)])
@pytest.mark.parametrize("affine", [True, False])
def test_groupnorm_fwd_bwd(dt, act, shape, groups, affine):
    rng = np.random.default_rng(17)
    c = shape[-2]
    x = prep(rng.standard_normal(shape) * rng.uniform(0.5, 2, (c, 1)), dt)
    g = prep(rng.uniform(0.5, 1.5, c), dt) if affine else None
    b = prep(rng.standard_normal(c) * 0.1, dt) if affine else None
    z_ref, pb_ref = O.groupnorm_rrule(x, g, b, groups, act, 1e-5)
    z, pb = L.rrule_groupnorm(dev(x, dt), dev(g, dt), dev(b, dt), groups, act, 1e-5)
    check(z, z_ref, dt, "y")
    delta = prep(rng.standard_normal(shape), dt)
    dx_ref, dg_ref, db_ref = pb_ref(delta)
    dx, dg, db = pb(dev(delta, dt))
    check(dx, dx_ref, dt, "dx", scale=delta)
    check(dg, dg_ref, dt, "dgamma")
    check(db, db_ref, dt, "dbeta")


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("act", ["identity", "relu"])
@pytest.mark.parametrize("shape", [(4, 4, 6, 2), (16, 16, 8, 3), (7, 5, 3), (64, 64, 4, 2)])
@pytest.mark.parametrize("affine", [True, False])
def test_instancenorm_all_modes(dt, act, shape, affine):
    # lib/LuxLib/test/normalization/instancenorm_tests.jl:18-80: without running statistics, with them in
    # training mode (updated statistics returned) and in test mode (statistics used as they are)
    rng = np.random.default_rng(21)
    c = shape[-2]
    x = prep(rng.standard_normal(shape) * 1.5 + 0.3, dt)
    g = prep(rng.uniform(0.5, 1.5, c), dt) if affine else None
    b = prep(rng.standard_normal(c) * 0.1, dt) if affine else None
    rm, rv = prep(rng.uniform(0, 1, c), dt), prep(rng.standard_normal(c) ** 2 + 0.1, dt)
    y_ref, _ = O.instancenorm(x, g, b, None, None, True, act, 0.1, 1e-5)
    y, stats = L.instancenorm(dev(x, dt), dev(g, dt), dev(b, dt), None, None, True, act, 0.1, 1e-5)
    check(y, y_ref, dt, "y")
    assert stats == (None, None)
    y_ref, (rm_ref, rv_ref) = O.instancenorm(x, g, b, rm, rv, True, act, 0.1, 1e-5)
    y, (nrm, nrv) = L.instancenorm(dev(x, dt), dev(g, dt), dev(b, dt), dev(rm, dt), dev(rv, dt), True, act, 0.1, 1e-5)
    check(y, y_ref, dt, "y (training, running statistics)")
    check(nrm, rm_ref, dt, "running_mean", tol=1e-5 if dt == "f32" else None)
    check(nrv, rv_ref, dt, "running_var", tol=1e-5 if dt == "f32" else None)
    y_ref, _ = O.instancenorm(x, g, b, rm, rv, False, act, 0.1, 1e-5)
    y, (srm, srv) = L.instancenorm(dev(x, dt), dev(g, dt), dev(b, dt), dev(rm, dt), dev(rv, dt), False, act, 0.1, 1e-5)
    check(y, y_ref, dt, "y (test mode)")
    check(srm, rm, dt, "running_mean unchanged")
    z_ref, pb_ref = O.instancenorm_rrule(x, g, b, act, 1e-5)
    z, pb = L.rrule_instancenorm(dev(x, dt), dev(g, dt), dev(b, dt), act, 1e-5)
    check(z, z_ref, dt, "z")
    delta = prep(rng.standard_normal(shape), dt)
    dx_ref, dg_ref, db_ref = pb_ref(delta)
    dx, dg, db = pb(dev(delta, dt))
    check(dx, dx_ref, dt, "dx", scale=delta)
    check(dg, dg_ref, dt, "dgamma")
    check(db, db_ref, dt, "dbeta")


def test_instancenorm_needs_three_dims():
    with pytest.raises(AssertionError):
        L.instancenorm(L.jl_zeros((4, 3), torch.float32, "cuda"), None, None)


def test_groupnorm_errors():
    x = L.jl_zeros((4, 4, 6, 2), torch.float32, "cuda")
    with pytest.raises(L.ArgumentError):
        L.groupnorm(x, None, None, 4)
    with pytest.raises(L.ArgumentError):
        L.groupnorm(x, torch.ones(5, device="cuda"), torch.ones(5, device="cuda"), 3)


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("act", ["identity", "tanh"])
@pytest.mark.parametrize("shape,nd", [((16, 7), 1), ((4096, 9), 1), ((4, 4, 6, 3), 3), ((100, 33), 1), ((6000, 4), 1),
                                      ((24576, 3), 1), ((1030, 5), 1),
                                      # many rows of 2048 / 4096 / 1152 elements: the warp-per-row forward of 2-byte rows
                                      ((2048, 2400), 1), ((4096, 2500), 1), ((1152, 2377), 1)])
@pytest.mark.parametrize("affine", [True, False])
def test_layernorm_fwd_bwd(dt, act, shape, nd, affine):
    rng = np.random.default_rng(18)
    x = prep(rng.standard_normal(shape) * 1.5 + 0.2, dt)
    # explicit dims: scale / bias carry the layer's shape (shape..., 1) (src/layers/normalize.jl:581-587)
    ashape = shape[:nd] + (1,) * (len(shape) - nd)
    g = prep(rng.uniform(0.5, 1.5, ashape), dt) if affine else None
    b = prep(rng.standard_normal(ashape) * 0.1, dt) if affine else None
    dims0 = tuple(range(nd))
    z_ref, pb_ref = O.layernorm_rrule(x, g, b, act, dims0, 1e-5)
    z, pb = L.rrule_layernorm(dev(x, dt), dev(g, dt), dev(b, dt), act, tuple(d + 1 for d in dims0), 1e-5)
    check(z, z_ref, dt, "y")
    delta = prep(rng.standard_normal(shape), dt)
    dx_ref, dg_ref, db_ref = pb_ref(delta)
    dx, dg, db = pb(dev(delta, dt))
    check(dx, dx_ref, dt, "dx", scale=delta)
    check(dg, dg_ref, dt, "dgamma")
    check(db, db_ref, dt, "dbeta")


def test_layernorm_dims_nothing_derives_rows_from_the_affine_rank():
    rng = np.random.default_rng(20)
    x = rng.standard_normal((48, 5)).astype(np.float32)
    g, b = rng.uniform(0.5, 1.5, 48).astype(np.float32), rng.standard_normal(48).astype(np.float32)
    y = L.layernorm(dev(x, "f32"), dev(g, "f32"), dev(b, "f32"), "identity", None, 1e-5)
    check(y, O.layernorm(x, g, b, "identity", None, 1e-5), "f32", "y")


def test_layernorm_property_and_errors():
    # lib/LuxLib/test/normalization/layernorm_tests.jl:54-57,100-113
    x = L.from_numpy(np.random.default_rng(19).standard_normal((4, 4, 6, 3)).astype(np.float32))
    y = L.to_numpy(L.layernorm(x, None, None, "identity", (1, 2, 3), 1e-5))
    assert np.allclose(y.mean(axis=(0, 1, 2)), 0, atol=1e-3) and np.allclose(y.std(axis=(0, 1, 2)), 1, atol=1e-3)
    with pytest.raises(L.ArgumentError):
        L.layernorm(x, None, None, "identity", None)
    with pytest.raises(AssertionError):
        s = torch.ones(4, 4, device="cuda")
        L.layernorm(x[:, :, 0, 0], s, s, "identity", None)


def test_float64_is_left_to_the_caller():
    x = torch.zeros(4, 4, dtype=torch.float64, device="cuda")
    with pytest.raises(L.LuxLibB200Error):
        L.fast_activation("relu", x)


# ------------------------------------------------------------------------------------------
# whole configurations, chained through the rrules (small versions of the benchmark configs)
# ------------------------------------------------------------------------------------------
def test_config_mlp_forward_backward_of_mse():
    """Dense(784 -> 256, relu) -> Dense(256 -> 10), Float32, batch 128, mean-squared error against one-hot targets:
    loss, and the gradients of both layers' parameters and of the input, against the CPU restatement."""
    rng = np.random.default_rng(0)
    W1, W2 = O.glorot_uniform(rng, (256, 784)), O.glorot_uniform(rng, (10, 256))
    b1, b2 = np.zeros(256, np.float32), np.zeros(10, np.float32)
    x = rng.standard_normal((784, 128)).astype(np.float32)
    t = np.zeros((10, 128), np.float32)
    t[rng.integers(0, 10, 128), np.arange(128)] = 1.0

    h_ref, pb1_ref = O.fused_dense_rrule("relu", W1, x, b1)
    y_ref, pb2_ref = O.fused_dense_rrule("identity", W2, h_ref, b2)
    loss_ref = np.mean((y_ref.astype(np.float64) - t) ** 2)
    dy_ref = (2.0 * (y_ref - t) / y_ref.size).astype(np.float32)
    dW2_ref, dh_ref, db2_ref = pb2_ref(dy_ref)
    dW1_ref, dx_ref, db1_ref = pb1_ref(dh_ref)

    h, pb1 = L.rrule_fused_dense("relu", dev(W1, "f32"), dev(x, "f32"), dev(b1, "f32"))
    y, pb2 = L.rrule_fused_dense("identity", dev(W2, "f32"), h, dev(b2, "f32"))
    check(y, y_ref, "f32", "y")
    tt = dev(t, "f32")
    loss = float(((y - tt).double() ** 2).mean())
    assert abs(loss - loss_ref) <= 1e-5 * abs(loss_ref)
    dy = 2.0 * (y - tt) / y.numel()
    dW2, dh, db2 = pb2(dy)
    dW1, dx, db1 = pb1(dh)
    for got, ref, name in ((dW2, dW2_ref, "dW2"), (db2, db2_ref, "db2"), (dW1, dW1_ref, "dW1"), (db1, db1_ref, "db1"),
                           (dx, dx_ref, "dx")):
        check(got, ref, "f32", name)


@pytest.mark.parametrize("dt", ["f32", "bf16"])
def test_config_conv_batchnorm_relu_block(dt):
    """Conv 3x3 64 -> 64 (stride 1, pad 1) -> BatchNorm(64) in training mode -> relu on a small WHCN input:
    output, running statistics and the gradients of x, filter, bias, gamma and beta."""
    rng = np.random.default_rng(2)
    x = prep(rng.standard_normal((16, 12, 64, 4)), dt)
    w = prep(O.kaiming_normal(rng, (3, 3, 64, 64)), dt)
    b = prep(np.zeros(64), dt)
    gam, bet = prep(np.ones(64), dt), prep(np.zeros(64), dt)
    rm, rv = prep(np.zeros(64), dt), prep(np.ones(64), dt)
    ocd, lcd = O.ConvDims.make(2, 1, 1, 1, 1, False), L.ConvDims.make(2, 1, 1, 1, 1, False)

    c_ref, pbc_ref = O.fused_conv_rrule("identity", w, x, b, ocd)
    c_in = prep(c_ref, dt)   # the conv output as the next op sees it in this storage type
    z_ref, (rm_ref, rv_ref), pbn_ref = O.batchnorm_rrule(c_in, gam, bet, rm, rv, True, "relu", 0.1, 1e-5)
    delta = prep(rng.standard_normal(z_ref.shape), dt)
    dc_ref, dg_ref, dbt_ref = pbn_ref(delta)
    dw_ref, dx_ref, db_ref = pbc_ref(prep(dc_ref, dt))

    c, pbc = L.rrule_fused_conv("identity", dev(w, dt), dev(x, dt), dev(b, dt), lcd)
    check(c, c_ref, dt, "conv")
    # the block's tail is judged on the reference's conv output so that storage rounding of c does not stack up
    z, (nrm, nrv), pbn = L.rrule_batchnorm(dev(c_in, dt), dev(gam, dt), dev(bet, dt), dev(rm, dt), dev(rv, dt), True,
                                           "relu", 0.1, 1e-5)
    check(z, z_ref, dt, "y")
    check(nrm, rm_ref, dt, "running_mean", tol=1e-5 if dt == "f32" else None)
    check(nrv, rv_ref, dt, "running_var", tol=1e-5 if dt == "f32" else None)
    dc, dg, dbt = pbn(dev(delta, dt))
    check(dg, dg_ref, dt, "dgamma")
    check(dbt, dbt_ref, dt, "dbeta")
    dw, dx, db = pbc(dev(prep(dc_ref, dt), dt))
    check(dw, dw_ref, dt, "dw")
    check(dx, dx_ref, dt, "dx")
    # BatchNorm's input gradient sums to zero over each channel, so the conv bias gradient is pure cancellation:
    # measured against the size of the terms that cancel
    check(db, db_ref, dt, "db", scale=np.abs(dc_ref).sum(axis=(0, 1, 3)), degenerate=True)
    assert L._cabi.load().lb2_poll_device_status(None) == 0


# ------------------------------------------------------------------------------------------
# optimiser step for a bucket of leaves (the update that follows the gradient all-reduce)
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("rule", ["descent", "momentum", "adam"])
def test_fused_optimizer_matches_the_rule_definitions(dt, rule):
    from luxlib_b200 import distributed as D
    rng = np.random.default_rng(31)
    shapes = [(33,), (64, 48), (3, 3, 8, 16), (5000,), (1,)] + [(17, 3)] * 60   # more leaves than one launch holds
    params = [prep(rng.standard_normal(s), dt) for s in shapes]
    opt = D.FusedOptimizer(D.NCCLBackend, rule, eta=0.05, rho=0.9, beta=(0.9, 0.999), eps=1e-8)
    dparams = [dev(p, dt) for p in params]
    states = opt.init(dparams)
    ostates = [O.optimiser_init(rule, p.astype(np.float64)) for p in params]
    oparams = [p.astype(np.float64) for p in params]
    for _ in range(3):
        grads = [prep(rng.standard_normal(s), dt) for s in shapes]
        opt.update(states, dparams, [dev(g, dt) for g in grads])
        for i, g in enumerate(grads):
            ostates[i], oparams[i] = O.optimiser_apply(rule, ostates[i], oparams[i], g.astype(np.float64), 0.05, 0.9,
                                                       (0.9, 0.999), 1e-8)
    for i in (0, 1, 2, 3, 4, 30, 64):
        check(dparams[i], oparams[i], dt, f"param {i}")


def test_fused_optimizer_master_copy_keeps_small_updates():
    # bf16 parameter 1.0 with updates of 1e-4: without an fp32 master copy every step rounds away
    from luxlib_b200 import distributed as D
    p = torch.ones(1024, device="cuda", dtype=torch.bfloat16)
    g = torch.ones(1024, device="cuda", dtype=torch.bfloat16)
    opt = D.FusedOptimizer(D.NCCLBackend, "descent", eta=1e-4, master=True)
    st = opt.init([p])
    for _ in range(100):
        opt.update(st, [p], [g])
    assert abs(float(st[0][2][0]) - 0.99) < 1e-5          # the master copy took all 100 steps
    assert abs(float(p[0]) - 0.99) < 4e-3                 # the parameter is its rounding


# ------------------------------------------------------------------------------------------
# pooling
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("kind", ["max", "mean"])
@pytest.mark.parametrize("shape,k,stride,pad", [((8, 8, 3, 2), (2, 2), None, 0), ((9, 7, 4, 3), (3, 3), (2, 2), 1),
                                                ((12, 10, 2, 2), (3, 2), (1, 2), (1, 2, 0, 1)), ((14, 5, 2), (3,), (2,), 1),
                                                ((6, 5, 4, 3, 2), (2, 2, 2), None, 0), ((7, 7, 8, 2), (7, 7), None, 0)])
def test_pooling_fwd_bwd(dt, kind, shape, k, stride, pad):
    rng = np.random.default_rng(33)
    x = prep(rng.standard_normal(shape), dt)
    y_ref, pb_ref = O.pool_rrule(kind, x, k, stride, pad)
    pd = L.PoolDims.make(k, stride, pad)
    y, pb = (L.rrule_maxpool if kind == "max" else L.rrule_meanpool)(dev(x, dt), pd)
    check(y, y_ref, dt, "y")
    dy = prep(rng.standard_normal(y_ref.shape), dt)
    check(pb(dev(dy, dt)), pb_ref(dy), dt, "dx")


def test_maxpool_ties_and_global_pools():
    x = L.jl_zeros((4, 4, 1, 1), torch.float32, "cuda")
    y, pb = L.rrule_maxpool(x, L.PoolDims.make((2, 2)))
    dx = L.to_numpy(pb(torch.ones_like(y)))
    assert dx[0, 0, 0, 0] == 1 and dx[1, 0, 0, 0] == 0 and dx[0, 1, 0, 0] == 0 and dx.sum() == 4
    xn = np.random.default_rng(34).standard_normal((5, 6, 3, 2)).astype(np.float32)
    xg = L.from_numpy(xn)
    np.testing.assert_allclose(L.to_numpy(L.meanpool(xg, L.PoolDims.global_(xg)))[0, 0], xn.mean(axis=(0, 1)), rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(L.to_numpy(L.maxpool(xg, L.PoolDims.global_(xg)))[0, 0], xn.max(axis=(0, 1)))
    assert L.PoolDims.adaptive(xg, (2, 3)).kernel == (3, 2)


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("act", ["identity", "relu", "gelu"])
def test_residual_add_activation(dt, act):
    # act.(x .+ y), the join of a residual block (perf/resnet/resnet.jl:6-7)
    rng = np.random.default_rng(35)
    x, y = prep(rng.standard_normal((9, 7, 5, 3)), dt), prep(rng.standard_normal((9, 7, 5, 3)), dt)
    s = prep(x + y, dt) if dt == "f32" else (x + y)   # the kernel adds in fp32
    z_ref = O.act_fn(act, s.astype(np.float32))
    z, pb = L.rrule_add_activation(act, dev(x, dt), dev(y, dt))
    check(z, z_ref, dt, "z")
    delta = prep(rng.standard_normal(x.shape), dt)
    dx, dy = pb(dev(delta, dt))
    ref = O.grad_activation(delta, prep(z_ref, dt), act, s.astype(np.float32))
    check(dx, ref, dt, "dx")
    check(dy, ref, dt, "dy")


# ------------------------------------------------------------------------------------------
# bounded device-side waits
# ------------------------------------------------------------------------------------------
def test_an_expired_device_side_wait_is_reported_and_leaves_the_device_usable():
    # Every mbarrier wait of the tensor-core kernels goes through one bounded wait routine. The self-test kernel runs
    # that routine on a barrier nothing arrives at, with a 1 ms limit: it must return (not hang), the status poll
    # must report the timeout exactly once, and the next operation must work.
    lib = L._cabi.load()
    assert lib.lb2_poll_device_status(None) == 0
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    assert lib.lb2_selftest_bounded_wait(1_000_000, torch.cuda.current_stream().cuda_stream) == 0
    t1.record()
    torch.cuda.synchronize()
    assert 0.5 <= t0.elapsed_time(t1) <= 50.0          # the wait ran for about its limit, then gave up
    assert lib.lb2_poll_device_status(None) == L._cabi.TIMEOUT
    assert b"0x40000000" in lib.lb2_last_error_string()
    assert lib.lb2_poll_device_status(None) == 0        # the poll cleared the word
    assert lib.lb2_selftest_bounded_wait(10, None) == L._cabi.BAD_ARG      # limits outside 1 us .. 100 ms are refused
    x = np.arange(12, dtype=np.float32).reshape(3, 4)
    check(L.fast_activation("relu", dev(x - 5, "f32")), np.maximum(x - 5, 0), "f32", "relu after the timeout")


# ------------------------------------------------------------------------------------------
# loss
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("shape", [(10, 128), (1000, 256), (7,), (3, 5, 2)])
def test_mse_loss_and_gradient(dt, shape):
    rng = np.random.default_rng(41)
    yh, y = prep(rng.standard_normal(shape), dt), prep(rng.standard_normal(shape), dt)
    l_ref, pb_ref = O.mse_loss_rrule(yh.astype(np.float64), y.astype(np.float64))
    l, pb = L.rrule_mse_loss(dev(yh, dt), dev(y, dt))
    check(l, np.array([l_ref]), "f32", "loss")          # the loss is a Float32 scalar for either storage type
    check(pb(), pb_ref(), dt, "dyhat")


# ------------------------------------------------------------------------------------------
# ConvTranspose (the data-gradient kernels as a forward operator)
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("act", ["identity", "relu", "gelu"])
@pytest.mark.parametrize("case", [
    # spatial, k, C_in, C_out, stride, pad, dilation, outpad, groups, flip, batch
    ((5, 4), (3, 3), 4, 6, 1, 0, 1, 0, 1, False, 2),
    ((7, 7), (3, 3), 64, 32, 2, 1, 1, 1, 1, False, 3),        # a decoder's 2x upsampling step (general tensor-core path)
    ((6, 5), (2, 2), 8, 8, 2, 0, 1, 0, 2, True, 2),           # groups: direct kernels
    ((14, 14), (3, 3), 128, 64, 1, 1, 1, 0, 1, False, 2),
])
def test_conv_transpose_fwd_bwd(dt, act, case):
    sp, k, cin, cu, stride, pad, dil, outpad, groups, flip, batch = case
    rng = np.random.default_rng(43)
    x = prep(rng.standard_normal(sp + (cin, batch)), dt)
    w = prep(O.kaiming_normal(rng, k + (cu // groups, cin)), dt)
    b = prep(rng.uniform(-0.1, 0.1, cu), dt)
    ocd = O.ConvDims.make(2, stride, pad, dil, groups, flip)
    lcd = L.ConvDims.make(2, stride, pad, dil, groups, flip)
    z_ref, pb_ref = O.conv_transpose_rrule(act, w, x, b, ocd, outpad, store=O.round_bf16 if dt == "bf16" else None)
    z, pb = L.rrule_conv_transpose(act, dev(w, dt), dev(x, dt), dev(b, dt), lcd, outpad)
    check(z, z_ref, dt, "y")
    delta = prep(rng.standard_normal(z_ref.shape), dt)
    dw_ref, dx_ref, db_ref = pb_ref(delta)
    dw, dx, db = pb(dev(delta, dt))
    check(dw, dw_ref, dt, "dw")
    check(dx, dx_ref, dt, "dx")
    check(db, db_ref, dt, "db")
    assert L._cabi.load().lb2_poll_device_status(None) == 0


# ------------------------------------------------------------------------------------------
# Scale layer
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("act", ["identity", "relu", "gelu", "tanh", "swish"])
@pytest.mark.parametrize("shape", [((5,), (5, 7)), ((8, 3), (8, 3, 33)), ((256,), (256, 130)), ((6, 4), (6, 4)), ((40, 8), (40, 8, 3, 70))])
@pytest.mark.parametrize("use_bias", [True, False])
def test_scale_layer_fwd_bwd(dt, act, shape, use_bias):
    dims, xs = shape
    rng = np.random.default_rng(45)
    x = prep(rng.standard_normal(xs), dt)
    w = prep(rng.uniform(0.5, 1.5, dims), dt)
    b = prep(rng.uniform(-0.3, 0.3, dims), dt) if use_bias else None
    z_ref, pb_ref = O.scale_rrule(act, w, x, b)
    z, pb = L.rrule_scale(act, dev(w, dt), dev(x, dt), dev(b, dt) if use_bias else None)
    check(z, z_ref, dt, "y")
    delta = prep(rng.standard_normal(xs), dt)
    dw_ref, dx_ref, db_ref = pb_ref(delta)
    dw, dx, db = pb(dev(delta, dt))
    check(dw, dw_ref, dt, "dw")
    check(dx, dx_ref, dt, "dx")
    if use_bias:
        check(db, db_ref, dt, "db")
    else:
        assert db is None


# ------------------------------------------------------------------------------------------
# cross-entropy loss
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("logits", [True, False])
@pytest.mark.parametrize("ls", [None, 0.15])
@pytest.mark.parametrize("shape", [(3, 5), (10, 128), (1000, 256), (37, 4, 6)])
def test_cross_entropy_loss_and_gradient(dt, logits, ls, shape):
    rng = np.random.default_rng(47)
    K = shape[0]
    cols = int(np.prod(shape[1:]))
    y = np.eye(K, dtype=np.float32)[:, rng.integers(0, K, cols)].reshape(shape)
    if logits:
        yhat = prep(rng.standard_normal(shape) * 2.0, dt)
    else:
        e = np.exp(rng.standard_normal(shape))
        yhat = prep(e / e.sum(axis=0, keepdims=True), dt)
    y = prep(y, dt)
    eps = float(np.finfo(np.float32).eps) if dt == "f32" else 2.0 ** -7      # eps(Float32) / eps(BFloat16)
    loss_ref, pb_ref = O.cross_entropy_rrule(yhat.astype(np.float64), y.astype(np.float64), logits=logits, label_smoothing=ls, epsilon=eps)
    loss, pb = L.rrule_cross_entropy_loss(dev(yhat, dt), dev(y, dt), logits=logits, label_smoothing=ls)
    got = float(loss.item())
    tol = 1e-5 if dt == "f32" else 1e-2
    err = abs(got - float(loss_ref)) / max(abs(float(loss_ref)), 1e-30)
    parity_report.record("loss", dt, err, tol)
    assert err <= tol, (got, float(loss_ref))
    check(pb(), pb_ref(), dt, "dyhat")


# ------------------------------------------------------------------------------------------
# batched matmul, scaled dot-product attention
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("shapes", [((4, 5, 6), (5, 3, 6)), ((70, 33, 5), (33, 130, 1)), ((64, 64), (64, 32, 9)), ((16, 8, 3, 2), (8, 12, 3, 2)),
                                    ((320, 300, 2), (300, 280, 2))])
def test_batched_matmul_fwd_bwd(dt, shapes):
    xs, ys = shapes
    rng = np.random.default_rng(49)
    x, y = prep(rng.standard_normal(xs), dt), prep(rng.standard_normal(ys), dt)
    z_ref, pb_ref = O.batched_matmul_rrule(x.astype(np.float64), y.astype(np.float64))
    z, pb = L.rrule_batched_matmul(dev(x, dt), dev(y, dt))
    check(z, z_ref, dt, "z")
    dz = prep(rng.standard_normal(z_ref.shape), dt)
    dx_ref, dy_ref = pb_ref(dz.astype(np.float64))
    dx, dy = pb(dev(dz, dt))
    check(dx, dx_ref, dt, "dx")
    check(dy, dy_ref, dt, "dy")


@pytest.mark.parametrize("dt", ["f32", "bf16"])
@pytest.mark.parametrize("variant", ["plain", "causal", "mask", "bias", "mask+bias4"])
@pytest.mark.parametrize("dims", [(8, 4, 2, 5, 7, 6, 3), (64, 8, 8, 128, 128, 64, 2), (32, 6, 2, 33, 65, 16, 1)])
def test_scaled_dot_product_attention_fwd_bwd(dt, variant, dims):
    D, H, Hkv, Lq, S, E, B = dims
    rng = np.random.default_rng(50)
    q = prep(rng.standard_normal((D, H, Lq, B)), dt)
    k = prep(rng.standard_normal((D, Hkv, S, B)), dt)
    v = prep(rng.standard_normal((E, Hkv, S, B)), dt)
    mask = bias = None
    causal = None
    if variant == "causal":
        causal = True
    if "mask" in variant:
        mask = rng.random((S, Lq)) > 0.3
        mask[0, :] = True                      # no column fully masked
    if variant == "bias":
        bias = prep(rng.standard_normal((S, Lq)) * 0.5, dt)
    if variant == "mask+bias4":
        bias = prep(rng.standard_normal((S, Lq, H, B)) * 0.5, dt)
    f64 = lambda a: None if a is None else a.astype(np.float64)
    (x_ref, w_ref), pb_ref = O.attention_rrule(f64(q), f64(k), f64(v), mask=mask, is_causal=causal, bias=f64(bias))
    tmask = None if mask is None else L.from_numpy(mask.astype(np.uint8), "cuda", torch.uint8)
    (x, w), pb = L.rrule_scaled_dot_product_attention(dev(q, dt), dev(k, dt), dev(v, dt), mask=tmask, is_causal=causal,
                                                       bias=None if bias is None else dev(bias, dt))
    check(w, w_ref, dt, "weights")
    check(x, x_ref, dt, "x")
    dx = prep(rng.standard_normal(x_ref.shape), dt)
    dq_ref, dk_ref, dv_ref, db_ref = pb_ref(f64(dx))
    dq, dk, dv, db = pb(dev(dx, dt))
    # bf16: the weights and the logits gradient are stored in bf16 between the launches, as the reference's arrays would be
    check(dq, dq_ref, dt, "dq")
    check(dk, dk_ref, dt, "dk")
    check(dv, dv_ref, dt, "dv")
    if bias is not None:
        check(db, db_ref, dt, "dbias")
    assert L._cabi.load().lb2_poll_device_status(None) == 0


# ------------------------------------------------------------------------------------------
# conv -> BatchNorm(act) with the statistics taken from the convolution's epilogue
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dt", ["bf16", "f32"])
@pytest.mark.parametrize("act", ["identity", "relu"])
@pytest.mark.parametrize("case", [
    # spatial, k, C_in, C_out, stride, pad, batch
    ((14, 14), (3, 3), 128, 128, 1, 1, 8),       # general tensor-core path: sums from the epilogue (bf16)
    ((28, 28), (3, 3), 128, 128, 2, 1, 6),       # strided; two epilogue halves of 64 channels
    ((9, 7), (3, 3), 128, 512, 2, 1, 5),         # two column tiles of 256: the grid is a multiple of the tile count
    ((9, 7), (1, 1), 64, 512, 2, 0, 5),          # short contraction: the plain pair
    ((30, 30), (7, 7), 3, 64, 2, 3, 4),          # the folded stem geometry: the plain pair
    ((16, 16), (3, 3), 64, 64, 1, 1, 4),         # the stride-1 64-channel fast case: sums by a separate pass
    ((6, 5), (3, 3), 4, 6, 1, 1, 3),             # CUDA-core kernels + separate pass
])
def test_conv_batchnorm_pair_with_sums_from_the_conv(dt, act, case):
    sp, k, cin, cout, stride, pad, batch = case
    rng = np.random.default_rng(51)
    x = prep(rng.standard_normal(sp + (cin, batch)), dt)
    w = prep(O.kaiming_normal(rng, k + (cin, cout)), dt)
    gam = prep(rng.uniform(0.5, 1.5, cout), dt)
    bet = prep(rng.standard_normal(cout) * 0.1, dt)
    rm, rv = prep(rng.standard_normal(cout) * 0.1, dt), prep(rng.uniform(0.5, 1.5, cout), dt)
    ocd, lcd = O.ConvDims.make(2, stride, pad, 1, 1, False), L.ConvDims.make(2, stride, pad, 1, 1, False)
    store = O.round_bf16 if dt == "bf16" else (lambda a: a)
    u_ref, pb_conv = O.fused_conv_rrule("identity", w, x, None, ocd)
    u_ref = store(u_ref)                       # the convolution's result as the arrays' element type holds it
    y_ref, (nrm_ref, nrv_ref), pb_bn = O.batchnorm_rrule(u_ref, gam, bet, rm, rv, True, act, 0.1, 1e-5)
    y, (nrm, nrv), pb = L.rrule_conv_batchnorm(act, dev(w, dt), dev(x, dt), lcd, dev(gam, dt), dev(bet, dt), dev(rm, dt), dev(rv, dt), 0.1, 1e-5)
    check(y, y_ref, dt, "y")
    check(nrm, nrm_ref, dt, "running_mean")
    check(nrv, nrv_ref, dt, "running_var")
    delta = prep(rng.standard_normal(y_ref.shape), dt)
    du_ref, dg_ref, db_ref = pb_bn(delta)
    dw_ref, dx_ref, _ = pb_conv(store(du_ref))
    dw, dx, dg, db = pb(dev(delta, dt))
    check(dg, dg_ref, dt, "dgamma")
    check(db, db_ref, dt, "dbeta")
    check(dw, dw_ref, dt, "dw")
    check(dx, dx_ref, dt, "dx")
    assert L._cabi.load().lb2_poll_device_status(None) == 0


@pytest.mark.parametrize("dt", ["bf16", "f32"])
@pytest.mark.parametrize("case", [((14, 14), (3, 3), 128, 128, 1, 1, 8), ((9, 7), (1, 1), 64, 512, 2, 0, 5), ((30, 30), (7, 7), 3, 64, 2, 3, 4),
                                  ((16, 16), (3, 3), 64, 64, 1, 1, 4), ((6, 5), (3, 3), 4, 6, 1, 1, 3)])
def test_conv_fwd_sums_entry_point_on_every_route(dt, case):
    # lb2_conv_fwd_sums itself (the Python pair takes it only where the epilogue form pays): y and the per-channel sums of
    # the stored y and y^2, from the epilogue on the general bf16 path and from lb2_channel_sums elsewhere
    import ctypes as C
    sp, k, cin, cout, stride, pad, batch = case
    rng = np.random.default_rng(52)
    x = prep(rng.standard_normal(sp + (cin, batch)), dt)
    w = prep(O.kaiming_normal(rng, k + (cin, cout)), dt)
    ocd, lcd = O.ConvDims.make(2, stride, pad, 1, 1, False), L.ConvDims.make(2, stride, pad, 1, 1, False)
    y_ref = O.conv(x.astype(np.float64), w.astype(np.float64), ocd)
    y_st = O.round_bf16(y_ref).astype(np.float64) if dt == "bf16" else y_ref.astype(np.float32).astype(np.float64)
    lib = L._cabi.load()
    X, W = dev(x, dt), dev(w, dt)
    from luxlib_b200 import ops as _ops
    d = _ops._conv_desc(W, X, lcd)
    y = L.jl_empty(y_ref.shape, X.dtype, "cuda")
    sums = torch.empty(2 * cout, dtype=torch.float32, device="cuda")
    dtc = 1 if dt == "bf16" else 0
    n = lib.lb2_conv_fwd_sums_workspace_bytes(C.byref(d), dtc)
    ws = torch.empty(max(n, 1), dtype=torch.uint8, device="cuda")
    rc = lib.lb2_conv_fwd_sums(y.data_ptr(), sums.data_ptr(), X.data_ptr(), W.data_ptr(), C.byref(d), dtc, 0, ws.data_ptr(), n, None)
    assert rc == 0, lib.lb2_last_error_string()
    check(y, y_ref, dt, "y")
    got = sums.cpu().numpy().reshape(cout, 2)
    # judged against the stored values the library itself produced (rounding of y differs from the oracle's by design)
    ys = L.to_numpy(y).astype(np.float64)
    axes = (0, 1, 3)
    s1, s2 = ys.sum(axis=axes), (ys * ys).sum(axis=axes)
    err2 = np.linalg.norm(got[:, 1] - s2) / np.linalg.norm(s2)
    err1 = np.linalg.norm(got[:, 0] - s1) / max(np.linalg.norm(s1), 1e-3 * np.sqrt(np.sum(np.abs(ys).sum(axis=axes) ** 2)))
    parity_report.record("sum y^2", dt, err2, 1e-5)
    parity_report.record("sum y", dt, err1, 1e-5, judged="against the sum of magnitudes when the sum cancels")
    assert err2 <= 1e-5 and err1 <= 1e-5, (err1, err2)
    del y_st
