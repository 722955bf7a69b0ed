"""Pins the CPU oracle: the reference's own known-answer tests, float64 finite
differences (the reference's gradient-truth method, lib/LuxTestUtils/src/autodiff.jl:147-294)
and an independent torch-CPU cross-check."""
import math

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import luxlib_oracle as O

ACTS = ["identity", "relu", "gelu", "tanh", "sigmoid", "swish"]


# ----------------------------------------------------------------------------
# Known-answer tests held by the reference for this path
# ----------------------------------------------------------------------------
def test_kat_batchnorm_values_and_running_stats():
    # test/core_layers/normalize_tests.jl:10-49
    x = np.array([[1, 3, 5], [2, 4, 6]], dtype=np.float32)
    g, b = np.ones(2, np.float32), np.zeros(2, np.float32)
    rm, rv = np.zeros(2, np.float32), np.ones(2, np.float32)
    y, (nrm, nrv) = O.batchnorm(x, g, b, rm, rv, True, "identity", 0.1, 1e-5)
    np.testing.assert_allclose(y, [[-1.22474, 0, 1.22474], [-1.22474, 0, 1.22474]], atol=1e-5)
    np.testing.assert_allclose(nrm, [0.3, 0.4], rtol=1e-6)
    expect = 0.1 * x.var(axis=1) * (3 / 2) + 0.9
    np.testing.assert_allclose(nrv, expect, rtol=1e-6)
    np.testing.assert_allclose(nrv, [1.3, 1.3], rtol=1e-6)
    yt, (rm2, rv2) = O.batchnorm(x, g, b, nrm, nrv, False, "identity", 0.1, 1e-5)
    assert abs(yt[0, 0] - (1 - 0.3) / math.sqrt(1.3)) < 1e-5
    assert rm2 is nrm and rv2 is nrv  # inference leaves the statistics untouched


def test_kat_dense_ones():
    # test/core_layers/basic_tests.jl:151-193
    W1, W2 = np.ones((1, 10), np.float32), np.ones((2, 10), np.float32)
    z1, z2 = np.zeros(1, np.float32), np.zeros(2, np.float32)
    assert (O.fused_dense_bias_activation("identity", W1, np.ones((10, 1), np.float32), z1) == 10).all()
    assert (O.fused_dense_bias_activation("identity", W1, np.ones((10, 2), np.float32), z1) == 10 * np.ones((1, 2))).all()
    x = np.concatenate([np.ones((10, 1)), 2 * np.ones((10, 1))], axis=1).astype(np.float32)
    assert (O.fused_dense_bias_activation("identity", W2, x, z2) == np.array([[10, 20], [10, 20]])).all()
    assert (O.fused_dense_bias_activation("identity", W2, x, None) == np.array([[10, 20], [10, 20]])).all()


def test_kat_conv_asymmetric_padding():
    # test/core_layers/conv_tests.jl:53-69
    x = np.ones((28, 28, 1, 1), np.float32)
    w = np.ones((3, 3, 1, 1), np.float32)
    cd = O.ConvDims.make(2, pad=(0, 1, 1, 2))
    y = O.fused_conv_bias_activation("relu", w, x, np.zeros(1, np.float32), cd)[:, :, 0, 0]
    assert y.shape == (27, 29)
    assert y[0, 0] == 6 and y[1, 1] == 9 and y[-1, 0] == 4
    assert y[0, -1] == 3 and y[0, -2] == 6 and y[-1, -1] == 2


@pytest.mark.parametrize("k", [(3, 3), (3, 1), (1, 3)])
def test_kat_conv_delta_image_reproduces_weight(k):
    # test/core_layers/conv_tests.jl:145-190 — the default is a true convolution
    rng = np.random.default_rng(0)
    x = np.zeros((7, 7, 1, 1), np.float32)
    x[3, 3, 0, 0] = 1
    w = rng.standard_normal(k + (1, 1)).astype(np.float32)
    y = O.conv(x, w, O.ConvDims.make(2))
    expect = np.zeros((7 - k[0] + 1, 7 - k[1] + 1, 1, 1), np.float32)
    r0 = slice(1, -1) if k[0] == 3 else slice(3, 4)
    r1 = slice(1, -1) if k[1] == 3 else slice(3, 4)
    expect[r0, r1, 0, 0] = w[:, :, 0, 0]
    np.testing.assert_allclose(y, expect, atol=1e-6)


def test_kat_layernorm_property():
    # lib/LuxLib/test/normalization/layernorm_tests.jl:54-57: mean≈0, std≈1 without affine
    rng = np.random.default_rng(1)
    x = rng.standard_normal((4, 4, 6, 3)).astype(np.float32)
    y = O.layernorm(x, None, None, "identity", dims=(0, 1, 2), eps=1e-5)
    assert np.allclose(y.mean(axis=(0, 1, 2)), 0, atol=1e-3)
    assert np.allclose(y.std(axis=(0, 1, 2)), 1, atol=1e-3)
    with pytest.raises(ValueError):
        O.layernorm(x, None, None, "identity", dims=None)
    with pytest.raises(AssertionError):
        O.layernorm(x[..., 0, 0], np.ones((4, 4), np.float32), np.ones((4, 4), np.float32), dims=None)


def test_fixed_array_generator():
    a = O.generate_fixed_array((2, 3))
    np.testing.assert_allclose(a, np.array([[1, 3, 5], [2, 4, 6]]) / 6, rtol=1e-7)


def test_default_epsilon():
    assert abs(O.default_epsilon(np.float32) - 1.1337e-5) < 1e-8
    assert abs(O.default_epsilon("bf16") - 0.03125) < 1e-9


def test_round_bf16_matches_torch():
    rng = np.random.default_rng(2)
    a = (rng.standard_normal(10000) * 10 ** rng.uniform(-6, 6, 10000)).astype(np.float32)
    ref = torch.from_numpy(a).to(torch.bfloat16).to(torch.float32).numpy()
    assert (O.round_bf16(a) == ref).all()


# ----------------------------------------------------------------------------
# finite differences in float64
# ----------------------------------------------------------------------------
def _fd(f, x, h=1e-6):
    g = np.zeros_like(x)
    it = np.nditer(x, flags=["multi_index"])
    for _ in it:
        i = it.multi_index
        old = x[i]
        x[i] = old + h
        fp = f()
        x[i] = old - h
        fm = f()
        x[i] = old
        g[i] = (fp - fm) / (2 * h)
    return g


@pytest.mark.parametrize("act", ACTS)
@pytest.mark.parametrize("gelu", ["tanh", "erf"])
def test_activation_derivative_fd(act, gelu):
    if act != "gelu" and gelu == "erf":
        pytest.skip("variant only matters for gelu")
    x = np.linspace(-4, 4, 41) + 0.013
    y = O.act_fn(act, x, gelu)
    d = O.act_grad(act, y, x, gelu)
    fd = (O.act_fn(act, x + 1e-6, gelu) - O.act_fn(act, x - 1e-6, gelu)) / 2e-6
    np.testing.assert_allclose(d, fd, atol=1e-7, rtol=1e-6)


@pytest.mark.parametrize("act", ACTS)
def test_dense_rrule_fd(act):
    rng = np.random.default_rng(3)
    W, x, b = rng.standard_normal((4, 5)), rng.standard_normal((5, 3)), rng.standard_normal(4)
    c = rng.standard_normal((4, 3))
    y, pb = O.fused_dense_rrule(act, W, x, b)
    dW, dx, db = pb(c)
    loss = lambda: float((O.fused_dense_bias_activation(act, W, x, b) * c).sum())
    np.testing.assert_allclose(dW, _fd(loss, W), atol=1e-6, rtol=1e-5)
    np.testing.assert_allclose(dx, _fd(loss, x), atol=1e-6, rtol=1e-5)
    np.testing.assert_allclose(db, _fd(loss, b), atol=1e-6, rtol=1e-5)


CONV_CASES = [
    # (spatial, k, cin, cout, stride, pad, dilation, groups, flip)  — shapes of lib/LuxLib/test/common_ops/conv_tests.jl:87-92
    ((4, 4), (3, 3), 4, 8, 1, 0, 1, 1, False),
    ((4, 4), (3, 3), 4, 8, 1, 0, 1, 2, False),
    ((5, 4), (3, 3), 4, 8, 2, (1, 1), 1, 1, False),
    ((6, 5), (3, 2), 2, 4, (2, 1), (0, 1, 1, 2), 1, 1, True),
    ((7,), (3,), 2, 4, 1, 1, 2, 1, False),
    ((4, 4, 3), (2, 2, 2), 2, 2, 1, 0, 1, 1, False),
]


@pytest.mark.parametrize("case", CONV_CASES)
def test_conv_rrule_fd(case):
    sp, k, cin, cout, stride, pad, dil, groups, flip = case
    rng = np.random.default_rng(4)
    nd = len(sp)
    cd = O.ConvDims.make(nd, stride, pad, dil, groups, flip)
    x = rng.standard_normal(sp + (cin, 2))
    w = rng.standard_normal(k + (cin // groups, cout))
    b = rng.standard_normal(cout)
    y, pb = O.fused_conv_rrule("gelu", w, x, b, cd)
    c = rng.standard_normal(y.shape)
    dw, dx, db = pb(c)
    loss = lambda: float((O.fused_conv_bias_activation("gelu", w, x, b, cd) * c).sum())
    np.testing.assert_allclose(dw, _fd(loss, w), atol=1e-6, rtol=1e-5)
    np.testing.assert_allclose(dx, _fd(loss, x), atol=1e-6, rtol=1e-5)
    np.testing.assert_allclose(db, _fd(loss, b), atol=1e-6, rtol=1e-5)


@pytest.mark.parametrize("act", ["identity", "relu", "swish"])
@pytest.mark.parametrize("affine", [True, False])
def test_batchnorm_rrule_fd(act, affine):
    rng = np.random.default_rng(5)
    x = rng.standard_normal((3, 2, 4, 3)) + 0.3
    g = rng.uniform(0.5, 1.5, 4) if affine else None
    b = rng.standard_normal(4) if affine else None
    rm, rv = np.zeros(4), np.ones(4)
    z, stats, pb = O.batchnorm_rrule(x, g, b, rm, rv, True, act, 0.1, 1e-5)
    c = rng.standard_normal(z.shape)
    dx, dg, db = pb(c)
    loss = lambda: float((O.batchnorm(x, g, b, rm, rv, True, act, 0.1, 1e-5)[0] * c).sum())
    np.testing.assert_allclose(dx, _fd(loss, x), atol=1e-6, rtol=1e-4)
    if affine:
        np.testing.assert_allclose(dg, _fd(loss, g), atol=1e-6, rtol=1e-5)
        np.testing.assert_allclose(db, _fd(loss, b), atol=1e-6, rtol=1e-5)


@pytest.mark.parametrize("shape,groups", [((6, 2), 2), ((4, 4, 6, 2), 3), ((2, 2, 6, 2), 2)])
@pytest.mark.parametrize("act", ["identity", "gelu"])
def test_groupnorm_rrule_fd(shape, groups, act):
    # shapes of lib/LuxLib/test/normalization/groupnorm_tests.jl:100
    rng = np.random.default_rng(6)
    x = rng.standard_normal(shape)
    g, b = rng.uniform(0.5, 1.5, shape[-2]), rng.standard_normal(shape[-2])
    z, pb = O.groupnorm_rrule(x, g, b, groups, act, 1e-5)
    c = rng.standard_normal(z.shape)
    dx, dg, db = pb(c)
    loss = lambda: float((O.groupnorm(x, g, b, groups, act, 1e-5) * c).sum())
    np.testing.assert_allclose(dx, _fd(loss, x), atol=1e-6, rtol=1e-4)
    np.testing.assert_allclose(dg, _fd(loss, g), atol=1e-6, rtol=1e-5)
    np.testing.assert_allclose(db, _fd(loss, b), atol=1e-6, rtol=1e-5)


@pytest.mark.parametrize("act", ["identity", "tanh"])
def test_layernorm_rrule_fd(act):
    rng = np.random.default_rng(7)
    x = rng.standard_normal((5, 3, 4))
    g, b = rng.uniform(0.5, 1.5, (5, 3)), rng.standard_normal((5, 3))
    z, pb = O.layernorm_rrule(x, g, b, act, None, 1e-5)
    c = rng.standard_normal(z.shape)
    dx, dg, db = pb(c)
    loss = lambda: float((O.layernorm(x, g, b, act, None, 1e-5) * c).sum())
    np.testing.assert_allclose(dx, _fd(loss, x), atol=1e-6, rtol=1e-4)
    np.testing.assert_allclose(dg, _fd(loss, g), atol=1e-6, rtol=1e-5)
    np.testing.assert_allclose(db, _fd(loss, b), atol=1e-6, rtol=1e-5)


# ----------------------------------------------------------------------------
# independent cross-check against torch CPU (stand-in for the vendor libraries
# the reference's GPU path would call)
# ----------------------------------------------------------------------------
def _to_torch_nchw(a):  # Julia (W,H,C,N) -> torch (N,C,H,W)
    return torch.from_numpy(np.ascontiguousarray(a.transpose(tuple(reversed(range(a.ndim))))))


def test_conv_matches_torch_cross_correlation_and_flip():
    rng = np.random.default_rng(8)
    x = rng.standard_normal((9, 8, 4, 2))
    w = rng.standard_normal((3, 3, 2, 6))
    xt, wt = _to_torch_nchw(x), _to_torch_nchw(w)  # weight -> (Cout, Cin/g, kH, kW)
    ref = F.conv2d(xt, wt, stride=(1, 2), padding=(1, 0), groups=2)  # torch order: (H, W)
    cd = O.ConvDims.make(2, stride=(2, 1), pad=(0, 0, 1, 1), groups=2, flipkernel=True)
    np.testing.assert_allclose(_to_torch_nchw(O.conv(x, w, cd)).numpy(), ref.numpy(), atol=1e-10)
    cd2 = O.ConvDims.make(2, stride=(2, 1), pad=(0, 0, 1, 1), groups=2, flipkernel=False)
    ref2 = F.conv2d(xt, torch.flip(wt, dims=(2, 3)), stride=(1, 2), padding=(1, 0), groups=2)
    np.testing.assert_allclose(_to_torch_nchw(O.conv(x, w, cd2)).numpy(), ref2.numpy(), atol=1e-10)


def test_norms_match_torch():
    rng = np.random.default_rng(9)
    x = rng.standard_normal((5, 4, 6, 3))
    g, b = rng.uniform(0.5, 1.5, 6), rng.standard_normal(6)
    xt = _to_torch_nchw(x)
    ref = F.group_norm(xt, 3, torch.from_numpy(g), torch.from_numpy(b), eps=1e-5)
    np.testing.assert_allclose(_to_torch_nchw(O.groupnorm(x, g, b, 3, "identity", 1e-5)).numpy(), ref.numpy(), atol=1e-10)
    rm, rv = torch.zeros(6, dtype=torch.float64), torch.ones(6, dtype=torch.float64)
    ref = F.batch_norm(xt, rm, rv, torch.from_numpy(g), torch.from_numpy(b), training=True, momentum=0.1, eps=1e-5)
    y, (nrm, nrv) = O.batchnorm(x, g, b, np.zeros(6), np.ones(6), True, "identity", 0.1, 1e-5)
    np.testing.assert_allclose(_to_torch_nchw(y).numpy(), ref.numpy(), atol=1e-10)
    np.testing.assert_allclose(nrm, rm.numpy(), atol=1e-12)
    np.testing.assert_allclose(nrv, rv.numpy(), atol=1e-12)
    x2 = rng.standard_normal((16, 7))
    g2, b2 = rng.uniform(0.5, 1.5, 16), rng.standard_normal(16)
    ref = F.layer_norm(torch.from_numpy(x2.T.copy()), (16,), torch.from_numpy(g2), torch.from_numpy(b2), 1e-5)
    np.testing.assert_allclose(O.layernorm(x2, g2, b2, "identity", None, 1e-5).T, ref.numpy(), atol=1e-10)


def test_instancenorm_matches_torch_and_the_running_statistics_rule():
    # independent cross-check of the restated generic normalization path (impl/normalization.jl:95-143)
    rng = np.random.default_rng(11)
    x = rng.standard_normal((5, 4, 6, 3))
    g, b = rng.uniform(0.5, 1.5, 6), rng.standard_normal(6)
    xt = _to_torch_nchw(x)
    rm0, rv0 = rng.uniform(0, 1, 6), rng.uniform(0.5, 2, 6)
    rm, rv = torch.from_numpy(rm0.copy()), torch.from_numpy(rv0.copy())
    ref = F.instance_norm(xt, rm, rv, torch.from_numpy(g), torch.from_numpy(b), use_input_stats=True, momentum=0.1, eps=1e-5)
    y, (nrm, nrv) = O.instancenorm(x, g, b, rm0, rv0, True, "identity", 0.1, 1e-5)
    np.testing.assert_allclose(_to_torch_nchw(y).numpy(), ref.numpy(), atol=1e-10)
    np.testing.assert_allclose(nrm, rm.numpy(), atol=1e-12)   # batch mean of per-sample means, S/(S-1) on the variance
    np.testing.assert_allclose(nrv, rv.numpy(), atol=1e-12)
    ref = F.instance_norm(xt, torch.from_numpy(rm0), torch.from_numpy(rv0), torch.from_numpy(g), torch.from_numpy(b),
                          use_input_stats=False, eps=1e-5)
    y, (srm, srv) = O.instancenorm(x, g, b, rm0, rv0, False, "identity", 0.1, 1e-5)
    np.testing.assert_allclose(_to_torch_nchw(y).numpy(), ref.numpy(), atol=1e-10)
    assert srm is rm0 and srv is rv0
    with pytest.raises(AssertionError):
        O.instancenorm(np.zeros((4, 3)), None, None, None, None, True)


@pytest.mark.parametrize("kind", ["max", "mean"])
@pytest.mark.parametrize("k,stride,pad", [((2, 2), None, 0), ((3, 3), (2, 2), 1), ((3, 2), (1, 2), (1, 0))])
def test_pooling_matches_torch(kind, k, stride, pad):
    # independent cross-check of the restated NNlib pooling (windows clipped, mean over the full window)
    rng = np.random.default_rng(12)
    x = rng.standard_normal((9, 8, 3, 2))
    y, pb = O.pool_rrule(kind, x, k, stride, pad)
    xt = _to_torch_nchw(x).requires_grad_(True)
    st = k if stride is None else stride
    pd = (pad, pad) if np.isscalar(pad) else pad
    # torch's kernel / stride / padding are (H, W); ours are (W, H)
    if kind == "max":
        ref = F.max_pool2d(xt, (k[1], k[0]), (st[1], st[0]), (pd[1], pd[0]))
    else:
        ref = F.avg_pool2d(xt, (k[1], k[0]), (st[1], st[0]), (pd[1], pd[0]), count_include_pad=True)
    np.testing.assert_allclose(_to_torch_nchw(y).numpy(), ref.detach().numpy(), atol=1e-12)
    dy = rng.standard_normal(y.shape)
    ref.backward(_to_torch_nchw(dy))
    np.testing.assert_allclose(_to_torch_nchw(pb(dy)).numpy(), xt.grad.numpy(), atol=1e-12)


def test_maxpool_gradient_goes_to_the_first_maximal_element():
    x = np.zeros((4, 4, 1, 1))
    y, pb = O.pool_rrule("max", x, (2, 2))
    dx = pb(np.ones_like(y))
    assert dx[0, 0, 0, 0] == 1 and dx[1, 0, 0, 0] == 0 and dx[0, 1, 0, 0] == 0 and dx.sum() == 4


def test_optimiser_rules_match_torch_optim():
    # Descent / Momentum / Adam as published for Optimisers.jl, against torch.optim on the same trajectory
    rng = np.random.default_rng(13)
    x0 = rng.standard_normal(50)
    grads = [rng.standard_normal(50) for _ in range(5)]
    for rule, make in (("descent", lambda p: torch.optim.SGD([p], lr=0.05)),
                       ("momentum", lambda p: torch.optim.SGD([p], lr=0.05, momentum=0.9)),
                       ("adam", lambda p: torch.optim.Adam([p], lr=0.05, betas=(0.9, 0.999), eps=1e-8))):
        p = torch.tensor(x0.copy(), requires_grad=True)
        opt = make(p)
        x, st = x0.copy(), O.optimiser_init(rule, x0)
        for g in grads:
            p.grad = torch.from_numpy(g.copy())
            opt.step()
            st, x = O.optimiser_apply(rule, st, x, g, 0.05, 0.9, (0.9, 0.999), 1e-8)
        np.testing.assert_allclose(x, p.detach().numpy(), rtol=1e-10, atol=1e-12)


def test_gelu_variants_match_torch():
    x = np.linspace(-5, 5, 101)
    np.testing.assert_allclose(O.act_fn("gelu", x, "tanh"), F.gelu(torch.from_numpy(x), approximate="tanh").numpy(), atol=1e-12)
    np.testing.assert_allclose(O.act_fn("gelu", x, "erf"), F.gelu(torch.from_numpy(x)).numpy(), atol=1e-12)
    np.testing.assert_allclose(O.act_fn("swish", x), F.silu(torch.from_numpy(x)).numpy(), atol=1e-12)


def test_mse_loss_against_torch_and_the_reference_docstring_example():
    # src/helpers/losses.jl:650-656: loss([1.1, 1.9, 3.1], 1:3) ≈ 0.01
    l, _ = O.mse_loss_rrule(np.array([1.1, 1.9, 3.1]), np.array([1.0, 2.0, 3.0]))
    assert abs(l - 0.01) < 1e-12
    import torch
    rng = np.random.default_rng(40)
    a, b = rng.standard_normal((10, 7)), rng.standard_normal((10, 7))
    ta = torch.tensor(a, requires_grad=True)
    lt = torch.nn.functional.mse_loss(ta, torch.tensor(b))
    lt.backward()
    l, pb = O.mse_loss_rrule(a, b)
    np.testing.assert_allclose(l, lt.item(), rtol=1e-12)
    np.testing.assert_allclose(pb(), ta.grad.numpy(), rtol=1e-12)


def test_conv_transpose_against_torch():
    # NNlib.conv_transpose = ∇conv_data (the ConvTranspose layer, src/layers/conv.jl:428-434); torch's
    # conv_transpose2d is the data gradient of a cross-correlation, i.e. the flipkernel = true case
    import torch
    rng = np.random.default_rng(42)
    for stride, pad, dil, outpad, groups in ((1, 0, 1, 0, 1), (2, 1, 1, 1, 1), (2, 1, 1, 0, 2), (3, 2, 2, 1, 1)):
        cin, cu = 4, 6
        x = rng.standard_normal((5, 4, cin, 2))
        w = rng.standard_normal((3, 3, cu // groups, cin))
        b = rng.standard_normal(cu)
        cd = O.ConvDims.make(2, stride, pad, dil, groups, True)
        z, pb = O.conv_transpose_rrule("identity", w, x, b, cd, outpad)
        tx = torch.tensor(np.ascontiguousarray(x.transpose(3, 2, 1, 0)), requires_grad=True)       # N, C, H, W
        tw = torch.tensor(np.ascontiguousarray(w.transpose(3, 2, 1, 0)), requires_grad=True)       # Cin, Cu/g, kH, kW
        tb = torch.tensor(b, requires_grad=True)
        tz = torch.nn.functional.conv_transpose2d(tx, tw, tb, stride=stride, padding=pad, output_padding=outpad, groups=groups, dilation=dil)
        np.testing.assert_allclose(z, tz.detach().numpy().transpose(3, 2, 1, 0), rtol=1e-10, atol=1e-10)
        delta = rng.standard_normal(z.shape)
        tz.backward(torch.tensor(np.ascontiguousarray(delta.transpose(3, 2, 1, 0))))
        dw, dx, db = pb(delta)
        np.testing.assert_allclose(dx, tx.grad.numpy().transpose(3, 2, 1, 0), rtol=1e-10, atol=1e-10)
        np.testing.assert_allclose(dw, tw.grad.numpy().transpose(3, 2, 1, 0), rtol=1e-10, atol=1e-10)
        np.testing.assert_allclose(db, tb.grad.numpy(), rtol=1e-10, atol=1e-10)


def test_scale_against_torch_autograd():
    import torch
    rng = np.random.default_rng(44)
    x, w, b = rng.standard_normal((5, 3, 7)), rng.standard_normal((5, 3)), rng.standard_normal((5, 3))
    delta = rng.standard_normal(x.shape)
    for act, tact in (("identity", lambda t: t), ("tanh", torch.tanh), ("relu", torch.relu), ("sigmoid", torch.sigmoid)):
        z, pb = O.scale_rrule(act, w, x, b)
        tx, tw, tb = (torch.tensor(a, requires_grad=True) for a in (x, w, b))
        tz = tact(tx * tw[..., None] + tb[..., None])
        tz.backward(torch.tensor(delta))
        dw, dx, db = pb(delta)
        np.testing.assert_allclose(z, tz.detach().numpy(), rtol=1e-12, atol=1e-12)
        np.testing.assert_allclose(dx, tx.grad.numpy(), rtol=1e-10, atol=1e-12)
        np.testing.assert_allclose(dw, tw.grad.numpy(), rtol=1e-10, atol=1e-12)
        np.testing.assert_allclose(db, tb.grad.numpy(), rtol=1e-10, atol=1e-12)
    z, pb = O.scale_rrule("identity", w, x, None)
    assert pb(delta)[2] is None and np.allclose(z, x * w[..., None])


def test_cross_entropy_known_answers_of_the_reference_docstring():
    # src/helpers/losses.jl:355-381: y one-hot 3x5, y_model = softmax(reshape(-7:7, 3, 5)); CrossEntropyLoss()(y_model, y)
    # ≈ 1.6076053, with label_smoothing = 0.15 ≈ 1.5776052, agg = sum gives 5x the mean
    z = np.arange(-7, 8, dtype=np.float32).reshape(5, 3).T          # Julia's column-major reshape
    y = np.array([[1, 0, 0, 0, 1], [0, 1, 0, 1, 0], [0, 0, 1, 0, 0]], dtype=np.float32)
    e = np.exp(z - z.max(axis=0, keepdims=True))
    y_model = (e / e.sum(axis=0, keepdims=True)).astype(np.float32)
    assert abs(float(y_model[0, 0]) - 0.0900306) < 1e-6 and abs(float(y_model[2, 0]) - 0.665241) < 1e-6
    assert abs(float(O.cross_entropy_rrule(y_model, y)[0]) - 1.6076053) < 2e-6
    assert abs(float(O.cross_entropy_rrule(y_model, y, label_smoothing=0.15)[0]) - 1.5776052) < 2e-6
    # the logits form on the logits themselves is the same loss (up to the epsilon of the probability form)
    assert abs(float(O.cross_entropy_rrule(z, y, logits=True)[0]) - 1.6076053) < 2e-6
    # gradients against torch autograd
    import torch
    rng = np.random.default_rng(46)
    zz = rng.standard_normal((7, 9))
    yy = np.eye(7)[:, rng.integers(0, 7, 9)]
    for ls in (None, 0.2):
        loss, pb = O.cross_entropy_rrule(zz, yy, logits=True, label_smoothing=ls)
        tz = torch.tensor(zz, requires_grad=True)
        yt = torch.tensor(yy if ls is None else (1 - ls) * yy + ls / 7)
        tl = -(yt * torch.log_softmax(tz, dim=0)).sum(dim=0).mean()
        tl.backward()
        assert abs(float(loss) - float(tl)) < 1e-12
        np.testing.assert_allclose(pb(), tz.grad.numpy(), rtol=1e-10, atol=1e-12)
    pp = np.abs(rng.standard_normal((7, 9))) + 0.1
    loss, pb = O.cross_entropy_rrule(pp, yy, logits=False, label_smoothing=0.1)
    tp = torch.tensor(pp, requires_grad=True)
    yt = torch.tensor(0.9 * yy + 0.1 / 7)
    tl = -(yt * torch.log(tp + np.finfo(np.float64).eps)).sum(dim=0).mean()
    tl.backward()
    assert abs(float(loss) - float(tl)) < 1e-12
    np.testing.assert_allclose(pb(), tp.grad.numpy(), rtol=1e-10, atol=1e-12)


def test_attention_and_batched_matmul_against_torch():
    import torch
    rng = np.random.default_rng(48)
    D, H, Hkv, L, S, E, B = 8, 4, 2, 5, 7, 6, 3
    q, k, v = rng.standard_normal((D, H, L, B)), rng.standard_normal((D, Hkv, S, B)), rng.standard_normal((E, Hkv, S, B))
    dx = rng.standard_normal((E, H, L, B))
    for causal in (False, True):
        (x, w), pb = O.attention_rrule(q, k, v, is_causal=causal or None)
        tq, tk, tv = (torch.tensor(np.ascontiguousarray(a.transpose(3, 1, 2, 0)), requires_grad=True) for a in (q, k, v))   # B, H, T, D
        kr, vr = tk.repeat_interleave(H // Hkv, dim=1), tv.repeat_interleave(H // Hkv, dim=1)
        am = torch.tensor(np.triu(np.ones((S, L), dtype=bool)).T) if causal else None                                      # (L, S): key s <= query l
        tx = torch.nn.functional.scaled_dot_product_attention(tq, kr, vr, attn_mask=am)
        tx.backward(torch.tensor(np.ascontiguousarray(dx.transpose(3, 1, 2, 0))))
        np.testing.assert_allclose(x, tx.detach().numpy().transpose(3, 1, 2, 0), rtol=1e-10, atol=1e-12)
        dq, dk, dv, _ = pb(dx)
        np.testing.assert_allclose(dq, tq.grad.numpy().transpose(3, 1, 2, 0), rtol=1e-9, atol=1e-12)
        np.testing.assert_allclose(dk, tk.grad.numpy().transpose(3, 1, 2, 0), rtol=1e-9, atol=1e-12)
        np.testing.assert_allclose(dv, tv.grad.numpy().transpose(3, 1, 2, 0), rtol=1e-9, atol=1e-12)
        assert np.allclose(w.sum(axis=0), 1.0)
    x3, y3 = rng.standard_normal((4, 5, 6)), rng.standard_normal((5, 3, 1))
    z, pb = O.batched_matmul_rrule(x3, y3)
    tx, ty = torch.tensor(x3.transpose(2, 0, 1).copy(), requires_grad=True), torch.tensor(y3.transpose(2, 0, 1).copy(), requires_grad=True)
    tz = torch.matmul(tx, ty)
    dz = rng.standard_normal(z.shape)
    tz.backward(torch.tensor(dz.transpose(2, 0, 1).copy()))
    np.testing.assert_allclose(z, tz.detach().numpy().transpose(1, 2, 0), rtol=1e-12)
    gx, gy = pb(dz)
    np.testing.assert_allclose(gx, tx.grad.numpy().transpose(1, 2, 0), rtol=1e-10)
    np.testing.assert_allclose(gy, ty.grad.numpy().transpose(1, 2, 0), rtol=1e-10)
