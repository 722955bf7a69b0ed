"""Parity at the benchmark configurations' full sizes. The CPU restatement cannot redo whole tensors of this
size in seconds, so each case checks size-independent pieces exactly: sampled output entries / rows / channels
recomputed in float64 from the same inputs (every output element of these operators depends on a slice of the
inputs that is cheap to recompute), plus the complete small outputs (bias, filter, scale gradients).
Tolerances are the contract's: rel-L2 1e-5 for Float32 storage, 1e-2 for bf16 storage."""
import numpy as np
import pytest
import torch

import luxlib_b200 as L
import parity_report
from oracle import luxlib_oracle as O

pytestmark = pytest.mark.gpu
TOL = {"f32": 1e-5, "bf16": 1e-2}
TDT = {"f32": torch.float32, "bf16": torch.bfloat16}


def rel(got, want, what="?", dt="?"):
    """plain rel-L2 against the float64 recomputation; recorded in the parity report under `what`"""
    got, want = np.asarray(got, np.float64).ravel(), np.asarray(want, np.float64).ravel()
    err = np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-300)
    parity_report.record(what, dt, err, TOL.get(dt, float("nan")))
    return err


def cm(t):
    """row-major bytes -> the Julia-shaped (column-major) view of the same memory"""
    return t.permute(*reversed(range(t.dim()))) if t.dim() > 1 else t


def host(t):
    """Julia-shaped float64 numpy copy of a device tensor"""
    return L.to_numpy(t).astype(np.float64)


def test_dense_config_full_size_sampled_entries():
    # W 4096x4096, x 4096x8192, bf16 storage, gelu: forward + dX + dW + db
    M, K, N = 4096, 4096, 8192
    g = torch.Generator(device="cuda").manual_seed(1)
    lim = (24.0 / (M + K)) ** 0.5
    W = cm(((torch.rand(K, M, device="cuda", generator=g) - 0.5) * lim).to(torch.bfloat16))
    x = cm(torch.randn(N, K, device="cuda", generator=g).to(torch.bfloat16))
    b = ((torch.rand(M, device="cuda", generator=g) - 0.5) * 0.2).to(torch.bfloat16)
    dy = cm(torch.randn(N, M, device="cuda", generator=g).to(torch.bfloat16))
    y, pb = L.rrule_fused_dense("gelu", W, x, b)
    dW, dx, db = pb(dy)
    assert L._cabi.load().lb2_poll_device_status(None) == 0
    Wn, xn, bn, dyn = host(W), host(x), host(b), host(dy)
    rng = np.random.default_rng(0)
    rows = rng.choice(M, 6, replace=False)
    cols = rng.choice(N, 6, replace=False)
    # rows of y, db and dW need the pre-activation of a whole row; columns of dx need a whole column of it
    pre_rows = Wn[rows] @ xn + bn[rows, None]                              # (6, N)
    y_rows = O.act_fn("gelu", pre_rows)
    g_rows = O.grad_activation(dyn[rows], y_rows, "gelu", pre_rows)        # (6, N)
    assert rel(host(y[rows.tolist()]), y_rows, "dense C2 y rows", "bf16") <= TOL["bf16"]
    assert rel(host(db)[rows], g_rows.sum(axis=1), "dense C2 db", "bf16") <= TOL["bf16"]
    assert rel(host(dW[rows.tolist()]), g_rows @ xn.T, "dense C2 dW rows", "bf16") <= TOL["bf16"]
    pre_cols = Wn @ xn[:, cols] + bn[:, None]                              # (M, 6)
    g_cols = O.grad_activation(dyn[:, cols], O.act_fn("gelu", pre_cols), "gelu", pre_cols)
    assert rel(host(dx[:, cols.tolist()]), Wn.T @ g_cols, "dense C2 dx cols", "bf16") <= TOL["bf16"]


@pytest.mark.parametrize("dt", ["bf16", "f32"])
def test_conv_config_full_size_sampled_entries(dt):
    # Conv 3x3 64 -> 64, stride 1, pad 1 on 56x56x64x256: forward (relu) + dx + dw + db
    Wd, Cc, Nb = 56, 64, 256
    g = torch.Generator(device="cuda").manual_seed(2)
    x = cm(torch.randn(Nb, Cc, Wd, Wd, device="cuda", generator=g).to(TDT[dt]))
    w = cm((torch.randn(Cc, Cc, 3, 3, device="cuda", generator=g) * (2.0 / 576) ** 0.5).to(TDT[dt]))
    b = ((torch.rand(Cc, device="cuda", generator=g) - 0.5) * 0.2).to(TDT[dt])
    dy = cm(torch.randn(Nb, Cc, Wd, Wd, device="cuda", generator=g).to(TDT[dt]))
    cd = L.ConvDims.make(2, 1, 1, 1, 1, False)
    y, pb = L.rrule_fused_conv("relu", w, x, b, cd)
    dw, dx, db = pb(dy)
    assert L._cabi.load().lb2_poll_device_status(None) == 0
    rng = np.random.default_rng(1)
    imgs = rng.choice(Nb, 3, replace=False)
    ocd = O.ConvDims.make(2, 1, 1, 1, 1, False)
    wn, bn = host(w), host(b)
    # whole images are independent of each other in the forward pass and in dx: redo three of them
    xs, dys = host(x[..., imgs.tolist()]), host(dy[..., imgs.tolist()])
    y_ref, pb_ref = O.fused_conv_rrule("relu", wn, xs, bn, ocd)
    _, dx_ref, _ = pb_ref(dys)
    assert rel(host(y[..., imgs.tolist()]), y_ref, "conv C3 y images", dt) <= TOL[dt]
    assert rel(host(dx[..., imgs.tolist()]), dx_ref, "conv C3 dx images", dt) <= TOL[dt]
    # db and dw contract over every image: g = dy * relu'(y) on the device output, reduced on the host in float64
    gn = host(dy) * (host(y) > 0)
    assert rel(host(db), gn.sum(axis=(0, 1, 3)), "conv C3 db", dt) <= TOL[dt]
    xn = host(x)
    xp = np.pad(xn, ((1, 1), (1, 1), (0, 0), (0, 0)))
    dw_ref = np.zeros((3, 3, Cc, Cc))
    for kw in range(3):
        for kh in range(3):
            # true convolution: y[i] += w[kw, kh] * x[i + pad - kw', ...] with kw' = flipped index (see the oracle's conv)
            win = xp[2 - kw:2 - kw + Wd, 2 - kh:2 - kh + Wd]               # (W, H, Cin, N) window paired with tap (kw, kh)
            dw_ref[kw, kh] = np.einsum("whcn,whdn->cd", win, gn, optimize=True)
    assert rel(host(dw), dw_ref, "conv C3 dw", dt) <= TOL[dt]


@pytest.mark.parametrize("dt", ["bf16", "f32"])
def test_batchnorm_config_full_size_channels(dt):
    # BatchNorm(64) + relu in training mode on 56x56x64x256 with running statistics
    shape = (256, 64, 56, 56)
    g = torch.Generator(device="cuda").manual_seed(3)
    x = cm((torch.randn(*shape, device="cuda", generator=g) * 1.3 + 0.2).to(TDT[dt]))
    dy = cm(torch.randn(*shape, device="cuda", generator=g).to(TDT[dt]))
    gam = (torch.rand(64, device="cuda", generator=g) + 0.5).to(TDT[dt])
    bet = (torch.randn(64, device="cuda", generator=g) * 0.1).to(TDT[dt])
    rm, rv = torch.zeros(64, device="cuda", dtype=TDT[dt]), torch.ones(64, device="cuda", dtype=TDT[dt])
    y, (nrm, nrv), pb = L.rrule_batchnorm(x, gam, bet, rm, rv, True, "relu", 0.1, 1e-5)
    dx, dg, db = pb(dy)
    assert L._cabi.load().lb2_poll_device_status(None) == 0
    chans = [0, 17, 63]
    # channels are independent: redo three of them as a 3-channel problem
    xs, dys = host(x[:, :, chans, :]), host(dy[:, :, chans, :])
    gs, bs = host(gam)[chans], host(bet)[chans]
    z_ref, (rm_ref, rv_ref), pb_ref = O.batchnorm_rrule(xs, gs, bs, np.zeros(3), np.ones(3), True, "relu", 0.1, 1e-5)
    dx_ref, dg_ref, db_ref = pb_ref(dys)
    assert rel(host(y[:, :, chans, :]), z_ref, "batchnorm C3 y channels", dt) <= TOL[dt]
    assert rel(host(nrm)[chans], rm_ref, "batchnorm C3 running_mean", dt) <= TOL[dt]
    assert rel(host(nrv)[chans], rv_ref, "batchnorm C3 running_var", dt) <= TOL[dt]
    assert rel(host(dx[:, :, chans, :]), dx_ref, "batchnorm C3 dx channels", dt) <= TOL[dt]
    assert rel(host(dg)[chans], dg_ref, "batchnorm C3 dgamma", dt) <= TOL[dt]
    assert rel(host(db)[chans], db_ref, "batchnorm C3 dbeta", dt) <= TOL[dt]


@pytest.mark.parametrize("dt", ["bf16", "f32"])
def test_layernorm_and_groupnorm_configs_full_size_rows(dt):
    g = torch.Generator(device="cuda").manual_seed(4)
    # LayerNorm over features on 4096 x 16384
    D, R = 4096, 16384
    x = cm((torch.randn(R, D, device="cuda", generator=g) * 1.3).to(TDT[dt]))
    dy = cm(torch.randn(R, D, device="cuda", generator=g).to(TDT[dt]))
    gam = (torch.rand(D, device="cuda", generator=g) + 0.5).to(TDT[dt])
    bet = (torch.randn(D, device="cuda", generator=g) * 0.1).to(TDT[dt])
    y, pb = L.rrule_layernorm(x, gam, bet, "identity", None, 1e-5)
    dx, dg, db = pb(dy)
    cols = [0, 5000, R - 1]
    z_ref, pb_ref = O.layernorm_rrule(host(x[:, cols]), host(gam), host(bet), "identity", None, 1e-5)
    dx_ref, _, _ = pb_ref(host(dy[:, cols]))
    assert rel(host(y[:, cols]), z_ref, "layernorm C4 y rows", dt) <= TOL[dt]
    assert rel(host(dx[:, cols]), dx_ref, "layernorm C4 dx rows", dt) <= TOL[dt]
    xn, dyn = host(x), host(dy)
    xh = (xn - xn.mean(axis=0)) / np.sqrt(xn.var(axis=0) + 1e-5)
    assert rel(host(dg), (dyn * xh).sum(axis=1), "layernorm C4 dgamma", dt) <= TOL[dt]
    assert rel(host(db), dyn.sum(axis=1), "layernorm C4 dbeta", dt) <= TOL[dt]
    del x, dy, y, dx, xn, dyn, xh
    # GroupNorm with 32 groups on 32x32x512x128
    shape = (128, 512, 32, 32)
    x = cm((torch.randn(*shape, device="cuda", generator=g) * (torch.rand(1, 512, 1, 1, device="cuda", generator=g) * 1.5 + 0.5)).to(TDT[dt]))
    dy = cm(torch.randn(*shape, device="cuda", generator=g).to(TDT[dt]))
    gam = (torch.rand(512, device="cuda", generator=g) + 0.5).to(TDT[dt])
    bet = (torch.randn(512, device="cuda", generator=g) * 0.1).to(TDT[dt])
    y, pb = L.rrule_groupnorm(x, gam, bet, 32, "identity", 1e-5)
    dx, dg, db = pb(dy)
    assert L._cabi.load().lb2_poll_device_status(None) == 0
    imgs = [0, 77, 127]
    z_ref, pb_ref = O.groupnorm_rrule(host(x[..., imgs]), host(gam), host(bet), 32, "identity", 1e-5)
    dx_ref, _, _ = pb_ref(host(dy[..., imgs]))
    assert rel(host(y[..., imgs]), z_ref, "groupnorm C4 y images", dt) <= TOL[dt]
    assert rel(host(dx[..., imgs]), dx_ref, "groupnorm C4 dx images", dt) <= TOL[dt]
    # the affine gradients sum over every sample: three channels of one group, all samples
    chans = [64, 70, 79]   # group 4 = channels 64..79
    xg, dyg = host(x[:, :, 64:80, :]), host(dy[:, :, 64:80, :])
    mu = xg.mean(axis=(0, 1, 2), keepdims=True)
    xh = (xg - mu) / np.sqrt(xg.var(axis=(0, 1, 2), keepdims=True) + 1e-5)
    idx = [c - 64 for c in chans]
    assert rel(host(dg)[chans], (dyg * xh).sum(axis=(0, 1, 3))[idx], "groupnorm C4 dgamma", dt) <= TOL[dt]
    assert rel(host(db)[chans], dyg.sum(axis=(0, 1, 3))[idx], "groupnorm C4 dbeta", dt) <= TOL[dt]
