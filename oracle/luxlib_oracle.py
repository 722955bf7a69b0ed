"""CPU restatement of LuxLib's fused-layer hot path (TEST INFRASTRUCTURE ONLY).

This module is the checker for the CUDA kernels. Only the test-suite, the smoke
check and the CPU-baseline leg of the benchmark may import it; the product path
never does.

It restates, in numpy, the arithmetic of LuxLib's own in-tree CPU code:

  dense        lib/LuxLib/src/impl/matmul.jl:73-83 (bias first, then C += A*B),
               lib/LuxLib/src/impl/dense.jl:46-57,71-113,290-291
  bias+act     lib/LuxLib/src/impl/bias_activation.jl:222-270, common_ops.jl:25-38
  activation   lib/LuxLib/src/impl/activation.jl:115-154 (sigma and Delta * sigma')
  conv         lib/LuxLib/src/impl/conv.jl:144-155,204-275
  batchnorm    lib/LuxLib/src/impl/normalization.jl:20-55,95-143,
               lib/LuxLib/src/impl/batchnorm.jl:149-176,212-227,517-570
  groupnorm    lib/LuxLib/src/impl/groupnorm.jl:5-22,174-206,477-533
  layernorm    lib/LuxLib/src/impl/layernorm.jl:3-14, normalization.jl:11-17
  mean_var     lib/LuxLib/src/impl/common_ops.jl:40-61

Third-party arithmetic that is NOT in the reference tree is restated from the
published definitions: NNlib (compat 0.9.33 in lib/LuxLib/Project.toml) supplies
`conv`, `∇conv_data`, `∇conv_filter` and the scalar activations. Convolution
semantics (true convolution = flipped kernel unless `flipkernel`, padding given as
(lo, hi) per spatial dim) are anchored on the reference's own layer tests
test/core_layers/conv_tests.jl:53-69 (asymmetric padding counts) and :145-190
(delta image reproduces the unflipped weight).

Parity status: pinned against every known-answer test the reference holds for
this path (BatchNorm values / running statistics, Dense ones-weights, the two conv
tests above, LayerNorm mean/std property). `gelu` is parity UNPINNED: the
reference tree does not contain NNlib's definition, so both the tanh form and the
erf form are provided and the same variant is always used on both sides.

Arrays use Julia's index order (W, H, C, N / features x batch); numpy memory
layout is irrelevant to the math here. All functions compute in the dtype of
their inputs (float32 or float64). bf16 rows are modelled as: inputs rounded to
bf16, math in float32, outputs rounded to bf16 (`round_bf16`).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional, Sequence, Tuple

import numpy as np

try:  # scipy is only needed for the exact-erf gelu variant
    from scipy.special import erf as _erf
except Exception:  # pragma: no cover
    _erf = np.vectorize(math.erf)

ACTIVATIONS = ("identity", "relu", "gelu", "tanh", "sigmoid", "swish")
# NNlib.fast_act aliases (src/layers/basic.jl:368): same function within the
# reference's own 1e-3 tolerance.
ALIASES = {"tanh_fast": "tanh", "sigmoid_fast": "sigmoid", "gelu_tanh": "gelu", "silu": "swish"}


def canonical_act(name: str) -> str:
    name = ALIASES.get(name, name)
    if name not in ACTIVATIONS:
        raise ValueError(f"unsupported activation {name!r}")
    return name


# --------------------------------------------------------------------------- #
# bf16 helpers
# --------------------------------------------------------------------------- #
def round_bf16(a: np.ndarray) -> np.ndarray:
    """Round float32 values to the nearest bfloat16 (ties to even), keep float32 storage."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    u = a.view(np.uint32)
    rounded = (u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) & np.uint32(0xFFFF0000)
    out = rounded.view(np.float32).copy()
    nan = np.isnan(a)
    if nan.any():
        out[nan] = np.nan
    return out.reshape(a.shape)


# --------------------------------------------------------------------------- #
# activations  (NNlib definitions; derivative forms as in
# lib/LuxLib/ext/SLEEFPiratesExt.jl:19-37 and NNlib's scalar rules)
# --------------------------------------------------------------------------- #
_GELU_A = 0.044715
_GELU_L = math.sqrt(2.0 / math.pi)


def _sigmoid(x):
    # numerically stable logistic
    out = np.empty_like(x)
    pos = x >= 0
    out[pos] = 1.0 / (1.0 + np.exp(-x[pos]))
    e = np.exp(x[~pos])
    out[~pos] = e / (1.0 + e)
    return out


def act_fn(name: str, x: np.ndarray, gelu: str = "tanh") -> np.ndarray:
    """sigma.(x)  — lib/LuxLib/src/impl/activation.jl:115-133."""
    name = canonical_act(name)
    T = x.dtype.type
    if name == "identity":
        return x.copy()
    if name == "relu":
        return np.maximum(x, T(0))
    if name == "tanh":
        return np.tanh(x)
    if name == "sigmoid":
        return _sigmoid(x)
    if name == "swish":
        return x * _sigmoid(x)
    if name == "gelu":
        if gelu == "tanh":
            inner = T(_GELU_L) * (x + T(_GELU_A) * x * x * x)
            return T(0.5) * x * (T(1) + np.tanh(inner))
        if gelu == "erf":
            return (T(0.5) * x * (T(1) + _erf(x / T(math.sqrt(2.0))))).astype(x.dtype)
        raise ValueError(gelu)
    raise AssertionError(name)


def act_grad(name: str, out: np.ndarray, pre: Optional[np.ndarray], gelu: str = "tanh") -> np.ndarray:
    """only_derivative(out, act, pre) — lib/LuxLib/src/utils.jl:84.

    `pre` may be None for the activations whose derivative needs the output only
    (lib/LuxLib/src/traits.jl:59-65): identity, relu, tanh, sigmoid.
    """
    name = canonical_act(name)
    T = out.dtype.type
    if name == "identity":
        return np.ones_like(out)
    if name == "relu":
        return (out > 0).astype(out.dtype)
    if name == "tanh":
        return T(1) - out * out
    if name == "sigmoid":
        return out * (T(1) - out)
    assert pre is not None, f"{name} needs the pre-activation"
    x = pre
    if name == "swish":
        s = _sigmoid(x)
        return out + s * (T(1) - out)
    if name == "gelu":
        if gelu == "tanh":
            inner = T(_GELU_L) * (x + T(_GELU_A) * x * x * x)
            t = np.tanh(inner)
            dinner = T(_GELU_L) * (T(1) + T(3 * _GELU_A) * x * x)
            return T(0.5) * (T(1) + t) + T(0.5) * x * (T(1) - t * t) * dinner
        if gelu == "erf":
            cdf = T(0.5) * (T(1) + _erf(x / T(math.sqrt(2.0))))
            pdf = np.exp(-T(0.5) * x * x) / T(math.sqrt(2.0 * math.pi))
            return (cdf + x * pdf).astype(out.dtype)
    raise AssertionError(name)


def needs_preactivation(name: str) -> bool:
    """True where sigma' needs x (gelu, swish): lib/LuxLib/src/traits.jl:67-69."""
    return canonical_act(name) in ("gelu", "swish")


def grad_activation(delta, out, name, pre, gelu="tanh"):
    """∇activation(Δ, out, act, x) = Δ .* σ′ — lib/LuxLib/src/impl/activation.jl:135-154."""
    if canonical_act(name) == "identity":
        return delta
    return delta * act_grad(name, out, pre, gelu)


# --------------------------------------------------------------------------- #
# bias + activation on the (S, C, B) view
# --------------------------------------------------------------------------- #
def _bias_shape(x: np.ndarray, b: np.ndarray):
    # reshaped_bias_dims: lib/LuxLib/src/impl/common_ops.jl:1-9
    if x.ndim == 1:
        return (b.shape[0],)
    shp = [1] * x.ndim
    shp[x.ndim - 2] = b.shape[0]
    return tuple(shp)


def bias_activation(act: str, x: np.ndarray, b: Optional[np.ndarray], gelu="tanh") -> np.ndarray:
    """σ.(x .+ b), b along dim N-1 — lib/LuxLib/src/impl/bias_activation.jl:222-270."""
    if b is not None:
        if x.ndim >= 2 and b.shape[0] != x.shape[x.ndim - 2]:
            raise ValueError("length(bias) must equal size(x, N-1)")  # api/bias_activation.jl:38-45
        x = x + b.reshape(_bias_shape(x, b))
    return act_fn(act, x, gelu)


def grad_bias_add(b: Optional[np.ndarray], delta: np.ndarray):
    """∇bias_add — lib/LuxLib/src/impl/common_ops.jl:25-38 (sum over all dims but N-1)."""
    if b is None:
        return None
    if delta.ndim == 1:
        return delta.copy()
    axes = tuple(i for i in range(delta.ndim) if i != delta.ndim - 2)
    return delta.sum(axis=axes, dtype=delta.dtype)


def bias_activation_rrule(act: str, x, b, gelu="tanh"):
    """rrule(bias_activation) — lib/LuxLib/src/impl/bias_activation.jl:55-141."""
    pre = x if b is None else x + b.reshape(_bias_shape(x, b))
    y = act_fn(act, pre, gelu)

    def pullback(delta):
        dx = grad_activation(delta, y, act, pre, gelu)
        return dx, grad_bias_add(b, dx)

    return y, pullback


# --------------------------------------------------------------------------- #
# dense
# --------------------------------------------------------------------------- #
def matmuladd(W, x, b):
    """lib/LuxLib/src/impl/matmul.jl:73-83: C .= bias ; C += A*B."""
    if W.shape[1] != x.shape[0]:
        raise ValueError("DimensionMismatch: size(W,2) != size(x,1)")  # matmul.jl:21-34
    y = W @ x
    if b is not None:
        if b.shape[0] != W.shape[0]:
            raise ValueError("DimensionMismatch: length(b) != size(W,1)")
        y = y + b[:, None]
    return y


def fused_dense_bias_activation(act: str, W, x, b, gelu="tanh"):
    """y = σ.(W*x .+ b) — lib/LuxLib/src/api/dense.jl:33-37, impl/dense.jl:4-57."""
    return act_fn(act, matmuladd(W, x, b), gelu)


def grad_matmul_bias(dy, W, x, b):
    """∇matmul_bias — lib/LuxLib/src/impl/dense.jl:290-291: (∂y·xᵀ, Wᵀ·∂y, Σ_cols ∂y)."""
    dW = dy @ x.T
    dx = W.T @ dy
    db = None if b is None else dy.sum(axis=1, dtype=dy.dtype)
    return dW, dx, db


def fused_dense_rrule(act: str, W, x, b, gelu="tanh"):
    """rrule(fused_dense) — lib/LuxLib/src/impl/dense.jl:71-113 (cases A and B)."""
    pre = matmuladd(W, x, b)
    y = act_fn(act, pre, gelu)

    def pullback(delta):
        dy = grad_activation(delta, y, act, pre if needs_preactivation(act) else None, gelu)
        return grad_matmul_bias(dy, W, x, b)

    return y, pullback


# --------------------------------------------------------------------------- #
# convolution (NNlib semantics restated; see module docstring)
# --------------------------------------------------------------------------- #
@dataclass
class ConvDims:
    """Fields NNlib.DenseConvDims is built from at src/layers/conv.jl:253-256."""
    stride: Tuple[int, ...]
    pad: Tuple[int, ...]          # (lo_1, hi_1, lo_2, hi_2, ...)
    dilation: Tuple[int, ...]
    groups: int = 1
    flipkernel: bool = False      # False = true convolution (kernel flipped); True = cross-correlation

    @staticmethod
    def make(nd: int, stride=1, pad=0, dilation=1, groups=1, flipkernel=False) -> "ConvDims":
        def tup(v, n):
            return tuple(int(q) for q in v) if isinstance(v, (tuple, list)) else (int(v),) * n
        s = tup(stride, nd)
        d = tup(dilation, nd)
        p = tup(pad, 2 * nd)
        if len(p) == nd:  # symmetric per-dim
            p = tuple(q for v in p for q in (v, v))
        assert len(s) == nd and len(d) == nd and len(p) == 2 * nd
        return ConvDims(s, p, d, int(groups), bool(flipkernel))


def conv_output_size(in_sz: Sequence[int], k: Sequence[int], cd: ConvDims):
    """src/layers/conv.jl:175-177: (in + pad_lo + pad_hi - dil*(k-1) - 1) ÷ stride + 1."""
    return tuple(
        (in_sz[i] + cd.pad[2 * i] + cd.pad[2 * i + 1] - cd.dilation[i] * (k[i] - 1) - 1) // cd.stride[i] + 1
        for i in range(len(k))
    )


def _kernel_offsets(k):
    return list(np.ndindex(*k))


def _tap(kidx, k, cd: ConvDims):
    """Position multiplier of each kernel index: true convolution visits x at
    (K-1-k)*dil, cross-correlation at k*dil."""
    return tuple((kidx[i] if cd.flipkernel else (k[i] - 1 - kidx[i])) * cd.dilation[i] for i in range(len(k)))


def conv(x: np.ndarray, w: np.ndarray, cd: ConvDims) -> np.ndarray:
    """NNlib.conv(x, w, cdims): x (spatial..., Cin, N), w (k..., Cin/groups, Cout)."""
    nd = x.ndim - 2
    k = w.shape[:nd]
    cin, n = x.shape[nd], x.shape[nd + 1]
    cin_g, cout = w.shape[nd], w.shape[nd + 1]
    g = cd.groups
    if cin_g * g != cin or cout % g != 0:
        raise ValueError("DimensionMismatch: channels / groups")
    osz = conv_output_size(x.shape[:nd], k, cd)
    padw = [(cd.pad[2 * i], cd.pad[2 * i + 1]) for i in range(nd)] + [(0, 0), (0, 0)]
    xp = np.pad(x, padw)
    y = np.zeros(osz + (cout, n), dtype=x.dtype)
    cog = cout // g
    for kidx in _kernel_offsets(k):
        off = _tap(kidx, k, cd)
        sl = tuple(slice(off[i], off[i] + cd.stride[i] * (osz[i] - 1) + 1, cd.stride[i]) for i in range(nd))
        xs = xp[sl]  # (osz..., Cin, N)
        for gi in range(g):
            xg = xs[..., gi * cin_g:(gi + 1) * cin_g, :]            # (o..., cin_g, N)
            wg = w[kidx][:, gi * cog:(gi + 1) * cog]                 # (cin_g, cog)
            # y[o..., co, n] += sum_ci xg[o..., ci, n] * wg[ci, co]
            y[..., gi * cog:(gi + 1) * cog, :] += np.einsum("...cn,cd->...dn", xg, wg, optimize=True)
    return y


def grad_conv_data(dy: np.ndarray, w: np.ndarray, cd: ConvDims, x_shape) -> np.ndarray:
    """NNlib.∇conv_data(∂y, w, cdims)."""
    nd = dy.ndim - 2
    k = w.shape[:nd]
    cin_g, cout = w.shape[nd], w.shape[nd + 1]
    g = cd.groups
    cog = cout // g
    osz = dy.shape[:nd]
    padded = tuple(x_shape[i] + cd.pad[2 * i] + cd.pad[2 * i + 1] for i in range(nd))
    dxp = np.zeros(padded + (x_shape[nd], x_shape[nd + 1]), dtype=dy.dtype)
    for kidx in _kernel_offsets(k):
        off = _tap(kidx, k, cd)
        sl = tuple(slice(off[i], off[i] + cd.stride[i] * (osz[i] - 1) + 1, cd.stride[i]) for i in range(nd))
        for gi in range(g):
            dyg = dy[..., gi * cog:(gi + 1) * cog, :]
            wg = w[kidx][:, gi * cog:(gi + 1) * cog]
            dxp[sl + (slice(gi * cin_g, (gi + 1) * cin_g), slice(None))] += np.einsum(
                "...dn,cd->...cn", dyg, wg, optimize=True)
    crop = tuple(slice(cd.pad[2 * i], cd.pad[2 * i] + x_shape[i]) for i in range(nd))
    return np.ascontiguousarray(dxp[crop])


def grad_conv_filter(x: np.ndarray, dy: np.ndarray, cd: ConvDims, w_shape) -> np.ndarray:
    """NNlib.∇conv_filter(x, ∂y, cdims)."""
    nd = x.ndim - 2
    k = tuple(w_shape[:nd])
    cin_g, cout = w_shape[nd], w_shape[nd + 1]
    g = cd.groups
    cog = cout // g
    osz = dy.shape[:nd]
    padw = [(cd.pad[2 * i], cd.pad[2 * i + 1]) for i in range(nd)] + [(0, 0), (0, 0)]
    xp = np.pad(x, padw)
    dw = np.zeros(tuple(w_shape), dtype=x.dtype)
    for kidx in _kernel_offsets(k):
        off = _tap(kidx, k, cd)
        sl = tuple(slice(off[i], off[i] + cd.stride[i] * (osz[i] - 1) + 1, cd.stride[i]) for i in range(nd))
        xs = xp[sl]
        for gi in range(g):
            xg = xs[..., gi * cin_g:(gi + 1) * cin_g, :]
            dyg = dy[..., gi * cog:(gi + 1) * cog, :]
            dw[kidx + (slice(None), slice(gi * cog, (gi + 1) * cog))] = np.einsum(
                "...cn,...dn->cd", xg, dyg, optimize=True)
    return dw


def fused_conv_bias_activation(act: str, w, x, b, cd: ConvDims, gelu="tanh"):
    """σ.(conv(x, w, cdims) .+ b) — lib/LuxLib/src/api/conv.jl:30-38, impl/conv.jl:144-155."""
    return bias_activation(act, conv(x, w, cd), b, gelu)


def fused_conv_rrule(act: str, w, x, b, cd: ConvDims, gelu="tanh"):
    """rrule(fused_conv) + ∇fused_conv — lib/LuxLib/src/impl/conv.jl:204-275."""
    pre = conv(x, w, cd)
    if b is not None:
        pre = pre + b.reshape(_bias_shape(pre, b))
    z = act_fn(act, pre, gelu)

    def pullback(delta):
        dy = grad_activation(delta, z, act, pre if needs_preactivation(act) else None, gelu)
        dw = grad_conv_filter(x, dy, cd, w.shape)
        dx = grad_conv_data(dy, w, cd, x.shape)
        db = grad_bias_add(b, dy)
        return dw, dx, db

    return z, pullback


def scale_rrule(act: str, w, x, b=None, gelu="tanh"):
    """Scale layer (src/layers/basic.jl:452-461): σ.(x .* weight .+ bias), weight / bias broadcast over the trailing
    batch dimensions of x. Pullback Δ -> (∂w, ∂x, ∂b) by the broadcast rule: g = Δ·σ′, ∂x = g·w, ∂w = Σ_batch g·x,
    ∂b = Σ_batch g."""
    nd = w.ndim
    wb = w.reshape(w.shape + (1,) * (x.ndim - nd))
    pre = x * wb
    if b is not None:
        pre = pre + b.reshape(wb.shape)
    z = act_fn(act, pre, gelu)

    def pullback(delta):
        g = grad_activation(delta, z, act, pre if needs_preactivation(act) else None, gelu)
        axes = tuple(range(nd, x.ndim))
        dw = (g * x).sum(axis=axes) if axes else g * x
        db = None if b is None else (g.sum(axis=axes) if axes else g)
        return dw, g * wb, db

    return z, pullback


def conv_transpose_output_size(in_sz, k, cd: ConvDims, outpad=0):
    """conv_transpose_dims (src/layers/conv.jl:19-45): (in - 1)*stride + 1 + (k - 1)*dil - pad_lo - pad_hi + outpad."""
    nd = len(in_sz)
    op = tuple(outpad) if isinstance(outpad, (tuple, list)) else (int(outpad),) * nd
    return tuple((in_sz[i] - 1) * cd.stride[i] + 1 + (k[i] - 1) * cd.dilation[i] - cd.pad[2 * i] - cd.pad[2 * i + 1] + op[i]
                 for i in range(nd))


def conv_transpose_rrule(act: str, w, x, b, cd: ConvDims, outpad=0, gelu="tanh", store=None):
    """ConvTranspose (src/layers/conv.jl:428-434): bias_activation!!(σ, conv_transpose(x, w, cdims), bias) with
    NNlib.conv_transpose(x, w, cdims) = ∇conv_data(x, w, cdims); w is (k..., C_out / groups, C_in).
    Pullback Δ -> (∂w, ∂x, ∂b): ∂x = conv(g, w), ∂w = ∇conv_filter(g, x).
    The layer is a composition of separate array operations, so the reference materialises conv_transpose's result and
    g = Δ .* act' in the arrays' element type before the next operation reads them; `store` is that rounding
    (round_bf16 for BFloat16 arrays, None for no rounding)."""
    store = store or (lambda a: a)
    nd = x.ndim - 2
    usz = conv_transpose_output_size(x.shape[:nd], w.shape[:nd], cd, outpad)
    u_shape = usz + (w.shape[nd] * cd.groups, x.shape[nd + 1])
    pre = store(grad_conv_data(x, w, cd, u_shape))
    if b is not None:
        pre = pre + b.reshape(_bias_shape(pre, b))
    z = act_fn(act, pre, gelu)

    def pullback(delta):
        g = store(grad_activation(delta, z, act, pre if needs_preactivation(act) else None, gelu))
        dx = conv(g, w, cd)
        dw = grad_conv_filter(g, x, cd, w.shape)
        db = grad_bias_add(b, g)
        return dw, dx, db

    return z, pullback


# --------------------------------------------------------------------------- #
# statistics
# --------------------------------------------------------------------------- #
def mean_var(x: np.ndarray, dims: Tuple[int, ...], corrected: bool = False):
    """lib/LuxLib/src/impl/common_ops.jl:40-43 (keepdims, like Julia's mean/var)."""
    mu = x.mean(axis=dims, keepdims=True, dtype=x.dtype)
    n = int(np.prod([x.shape[d] for d in dims]))
    var = ((x - mu) ** 2).sum(axis=dims, keepdims=True, dtype=x.dtype) / x.dtype.type(n - (1 if corrected else 0))
    return mu, var


def default_epsilon(dtype) -> float:
    """eps(T)^(5/7) — lib/LuxLib/src/utils.jl:130. 'bf16' → 0.03125."""
    if dtype == "bf16":
        return float(2.0 ** -7) ** (5.0 / 7.0)
    return float(np.finfo(dtype).eps) ** (5.0 / 7.0)


# --------------------------------------------------------------------------- #
# batchnorm
# --------------------------------------------------------------------------- #
def _bn_view(x: np.ndarray):
    # x viewed as (S, C, B): lib/LuxLib/src/impl/batchnorm.jl:90
    c, b = x.shape[-2], x.shape[-1]
    return x.reshape((-1, c, b), order="F") if x.ndim > 2 else x.reshape((1, c, b), order="F")


def batchnorm(x, gamma, beta, rmean, rvar, training: bool, act: str = "identity",
              momentum: float = 0.1, eps: float = 1e-5, gelu="tanh"):
    """LuxLib.batchnorm — lib/LuxLib/src/api/batchnorm.jl:31-55, impl/batchnorm.jl:29-49.

    Returns y, (running_mean′, running_var′) (None, None when no running stats).
    Statistics cases: lib/LuxLib/src/impl/normalization.jl:116-143.
    """
    y, stats, _ = batchnorm_full(x, gamma, beta, rmean, rvar, training, act, momentum, eps, gelu)
    return y, stats


def batchnorm_full(x, gamma, beta, rmean, rvar, training: bool, act: str = "identity",
                   momentum: float = 0.1, eps: float = 1e-5, gelu="tanh"):
    """As `batchnorm`, additionally returning the (μ, σ²) used for normalisation."""
    T = x.dtype.type
    x3 = _bn_view(x)
    S, C, B = x3.shape
    if (gamma is None) != (beta is None):
        raise ValueError("scale and bias must both be present or both be nothing")
    if training or rmean is None:
        mu = x3.mean(axis=(0, 2), dtype=x.dtype)
        var = ((x3 - mu[None, :, None]) ** 2).sum(axis=(0, 2), dtype=x.dtype) / T(S * B)
        if training and rmean is not None:
            # update_normalization_statistics: normalization.jl:95-110
            m = T(S * B)
            m1 = T(momentum)
            m2 = T(momentum) * m / (m - T(1))
            m3 = T(1) - m1
            new_rmean = m3 * rmean + m1 * mu
            new_rvar = m3 * rvar + m2 * var
        else:
            new_rmean, new_rvar = rmean, rvar
    else:
        mu, var = rmean.astype(x.dtype), rvar.astype(x.dtype)
        new_rmean, new_rvar = rmean, rvar
    # compute_batchnorm_scale_bias!: batchnorm.jl:149-176
    inv = T(1) / np.sqrt(var + T(eps))
    if gamma is None:
        g, bb = inv, -mu * inv
    else:
        g = gamma * inv
        bb = beta - mu * g
    y = act_fn(act, x3 * g[None, :, None] + bb[None, :, None], gelu).reshape(x.shape, order="F")
    return y, (new_rmean, new_rvar), (mu, var)


def batchnorm_rrule(x, gamma, beta, rmean, rvar, training: bool, act="identity",
                    momentum=0.1, eps=1e-5, gelu="tanh"):
    """Forward + pullback through Impl.batchnorm in training mode.

    ∇batchnorm_affine_normalize_cpu! (impl/batchnorm.jl:517-570) gives ∂x₁, ∂μ, ∂σ², ∂γ, ∂β;
    the mean_var rrule (common_ops.jl:45-61) then adds ∂μ/n + 2/n·∂σ²·(x-μ) to ∂x when the
    statistics were computed from the batch.
    """
    T = x.dtype.type
    y, new_stats, (mu, var) = batchnorm_full(x, gamma, beta, rmean, rvar, training, "identity", momentum, eps, gelu)
    z = act_fn(act, y, gelu)
    batch_stats = training or rmean is None
    x3 = _bn_view(x)
    S, C, B = x3.shape

    def pullback(delta):
        dy = grad_activation(delta, z, act, y, gelu)
        dy3 = _bn_view(dy)
        inv = T(1) / np.sqrt(var + T(eps))
        gp = inv if gamma is None else gamma * inv
        xmu = x3 - mu[None, :, None]
        dx1 = dy3 * gp[None, :, None]
        dmu = -dx1.sum(axis=(0, 2), dtype=x.dtype)
        dvar = -(dx1 * xmu).sum(axis=(0, 2), dtype=x.dtype) * T(0.5) * inv * inv
        if gamma is not None:
            dgamma = (dy3 * xmu).sum(axis=(0, 2), dtype=x.dtype) * inv
            dbeta = dy3.sum(axis=(0, 2), dtype=x.dtype)
        else:
            dgamma = dbeta = None
        dx = dx1
        if batch_stats:
            n = T(S * B)
            dx = dx1 + (dmu / n)[None, :, None] + (T(2) / n) * dvar[None, :, None] * xmu
        return dx.reshape(x.shape, order="F"), dgamma, dbeta

    return z, new_stats, pullback


# --------------------------------------------------------------------------- #
# groupnorm
# --------------------------------------------------------------------------- #
def groupnorm(x, gamma, beta, groups: int, act="identity", eps=1e-5, gelu="tanh"):
    """LuxLib.groupnorm — lib/LuxLib/src/api/groupnorm.jl:26-69, impl/groupnorm.jl:5-22,174-206."""
    y, _ = _groupnorm_fwd(x, gamma, beta, groups, act, eps, gelu)
    return y


def _gn_view(x, groups):
    c, n = x.shape[-2], x.shape[-1]
    if c % groups != 0:
        raise ValueError("number of channels must be divisible by groups")  # api/groupnorm.jl:40-67
    return x.reshape((-1, c // groups, groups, n), order="F")


def _groupnorm_fwd(x, gamma, beta, groups, act, eps, gelu):
    T = x.dtype.type
    c = x.shape[-2]
    if (gamma is None) != (beta is None):
        raise ValueError("scale and bias must both be present or both be nothing")
    if gamma is not None and (gamma.shape[0] != c or beta.shape[0] != c):
        raise ValueError("length(scale), length(bias) must equal the number of channels")
    x4 = _gn_view(x, groups)
    mu = x4.mean(axis=(0, 1), keepdims=True, dtype=x.dtype)
    var = ((x4 - mu) ** 2).mean(axis=(0, 1), keepdims=True, dtype=x.dtype)
    inv = T(1) / np.sqrt(var + T(eps))
    if gamma is None:
        pre = x4 * inv - mu * inv
    else:
        g4 = gamma.reshape((1, c // groups, groups, 1), order="F")
        b4 = beta.reshape((1, c // groups, groups, 1), order="F")
        gp = g4 * inv
        pre = x4 * gp + (b4 - mu * gp)
    y = act_fn(act, pre, gelu).reshape(x.shape, order="F")
    return y, (x4, mu, var, inv, pre)


def groupnorm_rrule(x, gamma, beta, groups: int, act="identity", eps=1e-5, gelu="tanh"):
    """∇groupnorm_affine_normalize_cpu! (impl/groupnorm.jl:477-533) chained through mean_var."""
    T = x.dtype.type
    c = x.shape[-2]
    z, (x4, mu, var, inv, pre) = _groupnorm_fwd(x, gamma, beta, groups, act, eps, gelu)

    def pullback(delta):
        dy = grad_activation(delta, z, act, pre.reshape(x.shape, order="F"), gelu)
        dy4 = _gn_view(dy, groups)
        xmu = x4 - mu
        if gamma is None:
            gp = inv
        else:
            gp = gamma.reshape((1, c // groups, groups, 1), order="F") * inv
        dx1 = dy4 * gp
        dmu = -dx1.sum(axis=(0, 1), keepdims=True, dtype=x.dtype)
        dvar = -(dx1 * xmu).sum(axis=(0, 1), keepdims=True, dtype=x.dtype) * T(0.5) * inv * inv
        n = T(x4.shape[0] * x4.shape[1])
        dx = dx1 + dmu / n + (T(2) / n) * dvar * xmu
        if gamma is not None:
            dgamma = (dy4 * xmu * inv).sum(axis=(0, 3), dtype=x.dtype).reshape(-1, order="F")
            dbeta = dy4.sum(axis=(0, 3), dtype=x.dtype).reshape(-1, order="F")
        else:
            dgamma = dbeta = None
        return dx.reshape(x.shape, order="F"), dgamma, dbeta

    return z, pullback


# --------------------------------------------------------------------------- #
# instancenorm
# --------------------------------------------------------------------------- #
def instancenorm(x, gamma, beta, rmean, rvar, training: bool, act="identity", momentum=0.1, eps=1e-5, gelu="tanh"):
    """LuxLib.instancenorm — lib/LuxLib/src/api/instancenorm.jl:32-77 through the generic
    `normalization` path (impl/normalization.jl:148-208) with reduce_dims = 1..N-2.

    Statistics per (channel, sample) unless running statistics are given and training is false
    (compute_batch_statistics, normalization.jl:116-143). In training mode with running statistics the
    per-sample statistics are averaged over the batch before the update, and the variance correction
    uses m = prod(size(x)[1:N-2]) (update_normalization_statistics, normalization.jl:95-110).
    Returns y, (running_mean', running_var')."""
    if x.ndim <= 2:
        raise AssertionError(f"`ndims(x) = {x.ndim}` must be at least > 2.")   # api/instancenorm.jl:72-75
    T = x.dtype.type
    c, b = x.shape[-2], x.shape[-1]
    if (gamma is None) != (beta is None):
        raise ValueError("scale and bias must both be present or both be nothing")
    x3 = x.reshape((-1, c, b), order="F")
    S = x3.shape[0]
    new_rmean, new_rvar = rmean, rvar
    if rmean is not None and not training:
        mu = rmean.astype(x.dtype)[None, :, None]
        var = rvar.astype(x.dtype)[None, :, None]
    else:
        mu = x3.mean(axis=0, keepdims=True, dtype=x.dtype)
        var = ((x3 - mu) ** 2).mean(axis=0, keepdims=True, dtype=x.dtype)
        if rmean is not None:
            mu_b = mu.mean(axis=2, dtype=x.dtype).reshape(-1)
            var_b = var.mean(axis=2, dtype=x.dtype).reshape(-1)
            m = T(S)
            m1 = T(momentum)
            m2 = T(momentum) * m / (m - T(1))
            m3 = T(1) - m1
            new_rmean = m3 * rmean + m1 * mu_b
            new_rvar = m3 * rvar + m2 * var_b
    # affine_normalize: normalization.jl:3-17
    if gamma is None:
        gp = T(1) / np.sqrt(var + T(eps))
        bp = -mu * gp
    else:
        gp = gamma[None, :, None] / np.sqrt(var + T(eps))
        bp = beta[None, :, None] - mu * gp
    y = act_fn(act, x3 * gp + bp, gelu).reshape(x.shape, order="F")
    return y, (new_rmean, new_rvar)


def instancenorm_rrule(x, gamma, beta, act="identity", eps=1e-5, gelu="tanh"):
    """Forward + pullback Δ -> (∂x, ∂scale, ∂bias) with per-instance statistics: the same arithmetic as
    groupnorm with one channel per group (the statistics of impl/normalization.jl:116-121 chained through
    the mean_var rule, impl/common_ops.jl:45-61)."""
    return groupnorm_rrule(x, gamma, beta, x.shape[-2], act, eps, gelu)


# --------------------------------------------------------------------------- #
# layernorm (row case: dims = leading dims, γ/β of the row shape or None)
# --------------------------------------------------------------------------- #
def layernorm(x, gamma, beta, act="identity", dims=None, eps=1e-5, gelu="tanh"):
    """LuxLib.layernorm — lib/LuxLib/src/api/layernorm.jl:32-43, impl/layernorm.jl:3-14.

    `dims` is a tuple of 0-based axes (Julia dims minus one); None with affine arrays of
    rank M means axes 0..N-M-1 (impl/layernorm.jl:24-30).
    """
    T = x.dtype.type
    if dims is None:
        if gamma is None:
            raise ValueError("`dims` must be passed explicitly if `scale` and `bias` are `nothing`")
        if not x.ndim > gamma.ndim:
            raise AssertionError("`x` must have more dimensions than `scale` and `bias`")
        dims = tuple(range(x.ndim - gamma.ndim))
        shp = gamma.shape + (1,) * (x.ndim - gamma.ndim)
        gamma, beta = gamma.reshape(shp, order="F"), beta.reshape(shp, order="F")
    mu, var = mean_var(x, tuple(dims), corrected=False)
    inv = T(1) / np.sqrt(var + T(eps))
    if gamma is None:
        pre = x * inv - mu * inv
    else:
        gp = gamma * inv
        pre = x * gp + (beta - mu * gp)
    return act_fn(act, pre, gelu)


def layernorm_rrule(x, gamma, beta, act="identity", dims=None, eps=1e-5, gelu="tanh"):
    """Standard LN gradient, i.e. what broadcast AD through affine_normalize + the mean_var
    rrule yields (impl/normalization.jl:11-17, common_ops.jl:45-61)."""
    T = x.dtype.type
    g, b = gamma, beta
    if dims is None:
        if gamma is None:
            raise ValueError("`dims` must be passed explicitly if `scale` and `bias` are `nothing`")
        dims = tuple(range(x.ndim - gamma.ndim))
        shp = gamma.shape + (1,) * (x.ndim - gamma.ndim)
        g, b = gamma.reshape(shp, order="F"), beta.reshape(shp, order="F")
    dims = tuple(dims)
    mu, var = mean_var(x, dims, corrected=False)
    inv = T(1) / np.sqrt(var + T(eps))
    xhat = (x - mu) * inv
    pre = xhat if g is None else xhat * g + b
    z = act_fn(act, pre, gelu)

    def pullback(delta):
        dy = grad_activation(delta, z, act, pre, gelu)
        gy = dy if g is None else dy * g
        m1 = gy.mean(axis=dims, keepdims=True, dtype=x.dtype)
        m2 = (gy * xhat).mean(axis=dims, keepdims=True, dtype=x.dtype)
        dx = inv * (gy - m1 - xhat * m2)
        if g is not None:
            red = tuple(i for i in range(x.ndim) if g.shape[i] == 1 and x.shape[i] != 1)
            dgamma = (dy * xhat).sum(axis=red, keepdims=True, dtype=x.dtype).reshape(gamma.shape, order="F")
            dbeta = dy.sum(axis=red, keepdims=True, dtype=x.dtype).reshape(beta.shape, order="F")
        else:
            dgamma = dbeta = None
        return dx, dgamma, dbeta

    return z, pullback


# --------------------------------------------------------------------------- #
# initialisers used to build the benchmark inputs
# (lib/WeightInitializers/src/initializers.jl:28-36, 97-104; utils.jl:6-10)
# --------------------------------------------------------------------------- #
def nfan(shape):
    if len(shape) == 1:
        return shape[0], shape[0]
    if len(shape) == 2:
        return shape[1], shape[0]
    rf = int(np.prod(shape[:-2]))
    return shape[-2] * rf, shape[-1] * rf


def glorot_uniform(rng: np.random.Generator, shape, gain=1.0, dtype=np.float32):
    fi, fo = nfan(shape)
    scale = gain * math.sqrt(24.0 / (fi + fo))
    return ((rng.random(shape, dtype=np.float64) - 0.5) * scale).astype(dtype)


def kaiming_normal(rng: np.random.Generator, shape, gain=math.sqrt(2.0), dtype=np.float32):
    fi, _ = nfan(shape)
    return (rng.standard_normal(shape) * (gain / math.sqrt(fi))).astype(dtype)


# --------------------------------------------------------------------------- #
# pooling (NNlib 0.9 direct CPU kernels, a dependency of the reference and not vendored; restated from
# its published behaviour: windows clipped to the input, mean over the full window size, the max-pool
# gradient to the first maximal element in (kw fastest, kh, kd) order). Call sites:
# src/layers/pooling.jl:42-57.
# --------------------------------------------------------------------------- #
def _pool_setup(x, kernel, stride, padding, dilation):
    nd = x.ndim - 2
    k = tuple(kernel)
    s = k if stride is None else ((stride,) * nd if np.isscalar(stride) else tuple(stride))
    d = (dilation,) * nd if np.isscalar(dilation) else tuple(dilation)
    p = (padding,) * (2 * nd) if np.isscalar(padding) else tuple(padding)
    if len(p) == nd:
        p = tuple(q for v in p for q in (v, v))
    out = tuple((x.shape[i] + p[2 * i] + p[2 * i + 1] - d[i] * (k[i] - 1) - 1) // s[i] + 1 for i in range(nd))
    return nd, k, s, d, p, out


def _pool_windows(x, kernel, stride, padding, dilation):
    """Yields (output index, list of input indices of the clipped window in kw-fastest order)."""
    import itertools
    nd, k, s, d, p, out = _pool_setup(x, kernel, stride, padding, dilation)
    for o in itertools.product(*[range(n) for n in reversed(out)]):
        o = tuple(reversed(o))
        win = []
        for kk in itertools.product(*[range(n) for n in reversed(k)]):
            kk = tuple(reversed(kk))   # last spatial dim slowest, first (w) fastest
            idx = tuple(o[i] * s[i] - p[2 * i] + kk[i] * d[i] for i in range(nd))
            if all(0 <= idx[i] < x.shape[i] for i in range(nd)):
                win.append(idx)
        yield o, win


def pool(kind: str, x, kernel, stride=None, padding=0, dilation=1):
    """maxpool / meanpool forward."""
    nd, k, s, d, p, out = _pool_setup(x, kernel, stride, padding, dilation)
    y = np.zeros(out + x.shape[-2:], dtype=x.dtype)
    T = x.dtype.type
    for o, win in _pool_windows(x, kernel, stride, padding, dilation):
        if kind == "max":
            vals = np.stack([x[i] for i in win]) if win else np.full((1,) + x.shape[-2:], -np.inf, x.dtype)
            y[o] = vals.max(axis=0)
        else:
            acc = np.zeros(x.shape[-2:], dtype=x.dtype)
            for i in win:
                acc = acc + x[i]
            y[o] = acc * T(1.0 / float(np.prod(k)))
    return y


def pool_rrule(kind: str, x, kernel, stride=None, padding=0, dilation=1):
    y = pool(kind, x, kernel, stride, padding, dilation)
    nd, k, s, d, p, out = _pool_setup(x, kernel, stride, padding, dilation)

    def pullback(dy):
        dx = np.zeros_like(x)
        T = x.dtype.type
        for o, win in _pool_windows(x, kernel, stride, padding, dilation):
            if kind == "max":
                taken = np.zeros(x.shape[-2:], dtype=bool)
                for i in win:
                    hit = (x[i] == y[o]) & ~taken
                    dx[i] += np.where(hit, dy[o], T(0))
                    taken |= hit
            else:
                for i in win:
                    dx[i] += dy[o] * T(1.0 / float(np.prod(k)))
        return dx

    return y, pullback


# --------------------------------------------------------------------------- #
# optimiser rules (Optimisers.jl 0.4.6 — a dependency of the reference, not vendored; restated from its
# published rule definitions: Descent, Momentum, Adam). State lives in the parameter's dtype.
# Call site: Optimisers.apply!(::DistributedOptimizer, ...) — src/distributed/public_api.jl:270-278.
# --------------------------------------------------------------------------- #
def optimiser_init(rule: str, x):
    if rule == "descent":
        return None
    if rule == "momentum":
        return np.zeros_like(x)
    if rule == "adam":
        return [np.zeros_like(x), np.zeros_like(x), 0]   # mt, vt, steps taken (beta^t carried implicitly)
    raise ValueError(rule)


def optimiser_apply(rule: str, state, x, dx, eta=1e-3, rho=0.9, beta=(0.9, 0.999), eps=1e-8):
    """One `apply!` + subtraction: returns (state', x'). Arithmetic in the array's dtype."""
    T = x.dtype.type
    if rule == "descent":
        return None, x - T(eta) * dx
    if rule == "momentum":
        v = T(rho) * state + T(eta) * dx
        return v, x - v
    if rule == "adam":
        mt, vt, t = state
        b1, b2 = T(beta[0]), T(beta[1])
        mt = b1 * mt + (T(1) - b1) * dx
        vt = b2 * vt + (T(1) - b2) * dx * dx
        t += 1
        b1t, b2t = T(1), T(1)
        for _ in range(t):
            b1t, b2t = b1t * b1, b2t * b2
        step = mt / (T(1) - b1t) / (np.sqrt(vt / (T(1) - b2t)) + T(eps)) * T(eta)
        return [mt, vt, t], x - step
    raise ValueError(rule)


def generate_fixed_array(shape, dtype=np.float32):
    """lib/LuxLib/test/shared_testsetup.jl:69-73: reshape((1:n)/n, sz) in column-major order."""
    n = int(np.prod(shape))
    return (np.arange(1, n + 1, dtype=np.float64) / n).astype(dtype).reshape(shape, order="F")


def rel_l2(a: np.ndarray, b: np.ndarray) -> float:
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    denom = np.linalg.norm(b.ravel())
    num = np.linalg.norm((a - b).ravel())
    return float(num / denom) if denom > 0 else float(num)


# --------------------------------------------------------------------------- #
# loss
# --------------------------------------------------------------------------- #
def batched_matmul_rrule(x, y):
    """batched_matmul for the default dimension roles (lib/LuxLib/src/api/batched_mul.jl:56-70): x (M, K, Bx...),
    y (K, N, By...) -> (M, N, B...), batch dimensions of size 1 repeated; matrices count as batch size 1.
    Pullback Δ -> (∂x, ∂y), summed over a repeated batch dimension."""
    x3 = x.reshape(x.shape + (1,)) if x.ndim == 2 else x
    y3 = y.reshape(y.shape + (1,)) if y.ndim == 2 else y
    z = np.einsum("mk...,kn...->mn...", x3, y3)

    def pullback(delta):
        dx = np.einsum("mn...,kn...->mk...", delta, np.broadcast_to(y3, y3.shape[:2] + delta.shape[2:]))
        dy = np.einsum("mk...,mn...->kn...", np.broadcast_to(x3, x3.shape[:2] + delta.shape[2:]), delta)
        for ax in range(2, delta.ndim):
            if x3.shape[ax] == 1 and delta.shape[ax] != 1:
                dx = dx.sum(axis=ax, keepdims=True)
            if y3.shape[ax] == 1 and delta.shape[ax] != 1:
                dy = dy.sum(axis=ax, keepdims=True)
        return dx.reshape(x.shape), dy.reshape(y.shape)

    return z, pullback


def attention_rrule(q, k, v, scale=None, mask=None, is_causal=None, bias=None):
    """scaled_dot_product_attention for head_dim = 1, token_dim = 3 (lib/LuxLib/src/impl/attention.jl:5-137):
    q (D, H, L, B), k (D, Hkv, S, B), v (E, Hkv, S, B); grouped keys / values repeated along the heads (repeat inner,
    :1-3, :47-51); logits[s, l, h, b] = sum_d k[d, h, s, b] * (q[d, h, l, b] / scale) (+ bias, masked with typemin:
    :120-128; causal mask = triu(trues(S, L)), :131-137); weights = softmax over s; x[e, h, l, b] = sum_s v[e, h, s, b] *
    weights[s, l, h, b]. Returns ((x, weights), Δx -> (∂q, ∂k, ∂v, ∂bias))."""
    D, H, L = q.shape[:3]
    Hkv, S = k.shape[1], k.shape[2]
    gs = H // Hkv
    kr, vr = np.repeat(k, gs, axis=1), np.repeat(v, gs, axis=1)
    sc = 1.0 / (np.sqrt(D) if scale is None else scale)
    logits = np.einsum("dhsb,dhlb->slhb", kr, q * sc)
    if bias is not None:
        logits = logits + (bias if bias.ndim == 4 else bias[:, :, None, None])
    keep = None
    if is_causal:
        keep = np.triu(np.ones((S, L), dtype=bool))[:, :, None, None]
    elif mask is not None:
        keep = mask.astype(bool) if mask.ndim == 4 else mask.astype(bool)[:, :, None, None]
    if keep is not None:
        logits = np.where(keep, logits, -np.inf)
    m = logits.max(axis=0, keepdims=True)
    e = np.exp(logits - m)
    w = e / e.sum(axis=0, keepdims=True)
    x = np.einsum("ehsb,slhb->ehlb", vr, w)

    def pullback(dx):
        dw = np.einsum("ehsb,ehlb->slhb", vr, dx)
        dvr = np.einsum("ehlb,slhb->ehsb", dx, w)
        dpre = w * (dw - (w * dw).sum(axis=0, keepdims=True))
        dq = np.einsum("dhsb,slhb->dhlb", kr, dpre) * sc
        dkr = np.einsum("dhlb,slhb->dhsb", q * sc, dpre)
        dk = dkr.reshape(D, Hkv, gs, S, -1).sum(axis=2)
        dv = dvr.reshape(v.shape[0], Hkv, gs, S, -1).sum(axis=2)
        db = None
        if bias is not None:
            db = dpre if bias.ndim == 4 else dpre.sum(axis=(2, 3))
        return dq, dk, dv, db

    return (x, w), pullback


def cross_entropy_rrule(yhat, y, logits=False, label_smoothing=None, epsilon=None):
    """CrossEntropyLoss(; dims = 1, agg = mean) — src/helpers/losses.jl:383-416. logits = true:
    mean(-sum(ỹ .* logsoftmax(ŷ; dims = 1); dims = 1)) (:408-412); logits = false: mean(-sum(xlogy.(ỹ, ŷ .+ ϵ); dims = 1))
    (:414-416) with ϵ = eps(T) unless given (:104-105); ỹ = (1 - α) y + α / size(y, 1) (label_smoothing, :172-177).
    Returns (loss, Δ -> ∂ŷ)."""
    K = yhat.shape[0]
    B = yhat.size // K
    yt = y if label_smoothing is None else (1 - label_smoothing) * y + label_smoothing / K
    yt = yt.astype(yhat.dtype)
    if logits:
        m = yhat.max(axis=0, keepdims=True)
        z = yhat - m
        lse = np.log(np.exp(z).sum(axis=0, keepdims=True))
        loss = -(yt * (z - lse)).sum() / B
        grad = (np.exp(z - lse) * yt.sum(axis=0, keepdims=True) - yt) / B
    else:
        eps = np.finfo(yhat.dtype).eps if epsilon is None else epsilon
        p = yhat + yhat.dtype.type(eps)
        with np.errstate(divide="ignore", invalid="ignore"):
            terms = np.where(yt == 0, 0.0, yt * np.log(p))
        loss = -terms.sum() / B
        grad = -yt / p / B

    def pullback(delta=1.0):
        return (grad * delta).astype(yhat.dtype)

    return yhat.dtype.type(loss), pullback


def mse_loss_rrule(yhat, y):
    """MSELoss() — src/helpers/losses.jl:659: GenericLossFunction(l2_distance_loss; agg = mean) with
    l2_distance_loss(x, y) = abs2(x - y) and derivative 2 (x - y) (src/helpers/losses.jl:121-125).
    Returns (loss, Δ -> ∂ŷ)."""
    d = yhat - y
    n = d.size
    loss = (d * d).sum(dtype=d.dtype) / d.dtype.type(n) if n else np.float32("nan")

    def pullback(delta=1.0):
        return (2.0 * d / n * delta).astype(d.dtype)

    return loss, pullback
