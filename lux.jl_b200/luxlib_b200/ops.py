"""Host-side mirror of the LuxLib operator API for the B200 path.

Same names, argument order and error behaviour as LuxLib's public ops
(lib/LuxLib/src/api/{dense,conv,batchnorm,groupnorm,layernorm,bias_activation,activation}.jl);
every op is one or two calls into libluxlib_b200.so through the C ABI. `rrule_*` functions mirror
the ChainRulesCore rules Zygote calls: they return the primal and a pullback closure.

Arrays are column-major device arrays (see arrays.py); activations are named by string
("identity", "relu", "gelu", "tanh", "sigmoid", "swish" and NNlib's *_fast aliases).
"""
from __future__ import annotations

import ctypes as C
import math
import warnings
from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

import torch

from . import _cabi
from ._cabi import ArgumentError, DimensionMismatch
from .arrays import as_colmajor, current_stream, dtype_code, jl_empty, jl_reshape, ptr, workspace

# --------------------------------------------------------------------------------------------
# activations
# --------------------------------------------------------------------------------------------
GELU_VARIANT = "tanh"  # which formula the name "gelu" denotes: "tanh" or "erf"

_ACT_CODES = {
    "identity": _cabi.ACT_IDENTITY, "relu": _cabi.ACT_RELU, "tanh": _cabi.ACT_TANH, "tanh_fast": _cabi.ACT_TANH,
    "sigmoid": _cabi.ACT_SIGMOID, "sigmoid_fast": _cabi.ACT_SIGMOID, "swish": _cabi.ACT_SWISH, "silu": _cabi.ACT_SWISH,
    "gelu_tanh": _cabi.ACT_GELU_TANH, "gelu_erf": _cabi.ACT_GELU_ERF,
}


def act_code(act: str) -> int:
    if act == "gelu":
        return _cabi.ACT_GELU_TANH if GELU_VARIANT == "tanh" else _cabi.ACT_GELU_ERF
    try:
        return _ACT_CODES[act]
    except KeyError:
        raise ArgumentError(f"activation {act!r} is not fused by the B200 path") from None


def needs_preactivation(act: str) -> bool:
    """activation_has_rrule but not activation_intermediate_not_needed
    (lib/LuxLib/src/traits.jl:59-69): gelu and swish need the pre-activation for their derivative."""
    return act_code(act) in (_cabi.ACT_GELU_TANH, _cabi.ACT_GELU_ERF, _cabi.ACT_SWISH)


# --------------------------------------------------------------------------------------------
# helpers
# --------------------------------------------------------------------------------------------
_warned_mixed = False


def _promote(*ts):
    """Mixed element types are promoted with a one-time warning (lib/LuxLib/ext/CUDAExt/cublaslt.jl:46-64)."""
    global _warned_mixed
    present = [t for t in ts if t is not None]
    dt = present[0].dtype
    for t in present[1:]:
        dt = torch.promote_types(dt, t.dtype)
    if any(t.dtype != dt for t in present):
        if not _warned_mixed:
            warnings.warn("Mixed-precision inputs: promoting to " + str(dt), stacklevel=3)
            _warned_mixed = True
        ts = tuple(None if t is None else t.to(dt) for t in ts)
    return ts


def _matrix_ld(t: torch.Tensor) -> Tuple[torch.Tensor, int]:
    """A column-major matrix and its leading dimension; copies when the first index is not contiguous."""
    if t.dim() != 2:
        raise DimensionMismatch(f"expected a matrix, got {t.dim()} dims")
    m, n = t.shape
    if t.numel() == 0:
        return t, max(m, 1)
    if t.stride(0) == 1 and (n == 1 or t.stride(1) >= max(m, 1)):
        return t, (t.stride(1) if n > 1 else max(m, 1))
    if m == 1 and n >= 1 and t.stride(1) >= 1:
        return t, t.stride(1)
    t = as_colmajor(t.contiguous() if not t.is_contiguous() else t)
    return t, max(m, 1)


def _ws(nbytes: int, device):
    w = workspace(nbytes, device)
    return w, ptr(w), int(nbytes) if w is not None else 0


# --------------------------------------------------------------------------------------------
# dense
# --------------------------------------------------------------------------------------------
def _dense_fwd(act: str, weight, x, b, want_preact: bool, flags: int = 0):
    lib = _cabi.load()
    weight, x, b = _promote(weight, x, b)
    if weight.dim() != 2:
        raise DimensionMismatch("weight must be a matrix")
    vec_in = x.dim() == 1
    if vec_in:  # a vector is one column (lib/LuxLib/src/impl/matmul.jl:3-5)
        x = x.reshape(-1, 1)
    M, K = weight.shape
    if x.shape[0] != K:
        raise DimensionMismatch(f"size(weight, 2) = {K} does not match size(x, 1) = {x.shape[0]}")
    if b is not None and b.shape[0] != M:
        raise DimensionMismatch(f"length(b) = {b.shape[0]} does not match size(weight, 1) = {M}")
    N = x.shape[1]
    W, ldw = _matrix_ld(weight)
    X, ldx = _matrix_ld(x)
    dt = dtype_code(W.dtype)
    y = jl_empty((M, N), W.dtype, W.device)
    pre = jl_empty((M, N), W.dtype, W.device) if want_preact else None
    _, wsp, wsn = _ws(lib.lb2_dense_fwd_workspace_bytes(M, N, K, dt, flags), W.device)
    _cabi.check(lib.lb2_dense_fwd(ptr(y), ptr(pre), ptr(W), ptr(X), ptr(b), M, N, K, ldw, ldx, max(M, 1), dt,
                                  act_code(act), flags, wsp, wsn, current_stream(W.device)))
    if vec_in:
        y = y.reshape(-1)
        pre = None if pre is None else pre.reshape(-1)
    return y, pre, (W, ldw, X, ldx, b, M, N, K, dt)


def fused_dense_bias_activation(act: str, weight, x, b=None, *, flags: int = 0):
    """y = act.(weight * x .+ b) — lib/LuxLib/src/api/dense.jl:33-37."""
    return _dense_fwd(act, weight, x, b, False, flags)[0]


def rrule_fused_dense(act: str, weight, x, b=None, *, flags: int = 0):
    """rrule(fused_dense) — lib/LuxLib/src/impl/dense.jl:71-113. Returns y and a pullback
    Δ -> (∂weight, ∂x, ∂b); the pre-activation is cached only for gelu / swish (case B)."""
    lib = _cabi.load()
    keep_pre = needs_preactivation(act)
    y, pre, (W, ldw, X, ldx, bb, M, N, K, dt) = _dense_fwd(act, weight, x, b, keep_pre, flags)
    code = act_code(act)

    def pullback(delta, on_param_grads=None, shadows=None, param_panels=1, mark=None, dx_reserve_sms=0):
        """Δ -> (∂weight, ∂x, ∂b).

        `on_param_grads(dW_panel, db_or_None)` switches to the data-parallel order of work: g = Δ .* act' and ∂b first,
        then ∂weight in `param_panels` column panels, then ∂x; the callback runs as soon as a panel is enqueued (∂b
        comes with the last one), so the caller's all-reduce of panel i runs underneath the GEMM of panel i+1 and the
        last panel's underneath the ∂x GEMM — a panel of 1024 columns is one wave of 256 x 256 tiles on 64 of the 74
        SM pairs, which leaves SMs to the collective, and `dx_reserve_sms` keeps that many SMs out of the ∂x GEMM for
        the same reason. Same kernels, more C calls. `mark()`, when given, is called after each phase (profiling
        hooks). `shadows = (dW, dx, db)` switches to the accumulate contract of the Enzyme rules: the gradients are
        added to those arrays in place and Δ is zeroed."""
        if on_param_grads is not None:
            d = as_colmajor(delta.reshape(M, N).to(W.dtype))
            g = jl_empty((M, N), W.dtype, W.device)
            db = jl_empty((M,), W.dtype, W.device) if bb is not None else None
            y2, pre2 = y.reshape(M, N), (None if pre is None else pre.reshape(M, N))
            _, wsp, wsn = _ws(lib.lb2_bias_act_bwd_workspace_bytes(1, M, N), W.device)
            _cabi.check(lib.lb2_bias_act_bwd(ptr(g), ptr(db), ptr(d), None if keep_pre else ptr(y2), ptr(pre2), 1, M, N, dt,
                                             code, wsp, wsn, current_stream(W.device)))
            if mark is not None:
                mark()
            dW = jl_empty((M, K), W.dtype, W.device)
            panels = max(1, min(int(param_panels), K))
            bounds = [K * i // panels for i in range(panels + 1)]
            for i in range(panels):
                k0, k1 = bounds[i], bounds[i + 1]
                matmul(g, X[k0:k1, :], transB=True, flags=flags, out=dW[:, k0:k1])      # g * x[k0:k1, :]'
                on_param_grads(dW[:, k0:k1], db if i == panels - 1 else None)
            if mark is not None:
                mark()
            dx = matmul(W, g, transA=True, flags=flags | _cabi.flag_reserve_sms(int(dx_reserve_sms)))      # W' * g
            if mark is not None:
                mark()
            return dW, (dx.reshape(x.shape) if x.dim() == 1 else dx), db
        d = as_colmajor(delta.reshape(M, N).to(W.dtype))
        if shadows is not None:
            # Enzyme's reverse pass (lib/LuxLib/src/impl/dense.jl:253-283): the gradients are ADDED to the caller's
            # shadow arrays (mul!(dW, g, x', true, true); db .+= ...) and the output shadow is zeroed afterwards.
            dW, dx, db = shadows
            dW, ldw_s = _matrix_ld(dW)
            dx2, ldx_s = _matrix_ld(dx.reshape(K, N))
            if (ldw_s, ldx_s) != (ldw, ldx):
                raise DimensionMismatch("shadow arrays must have the layout of weight and x")
        else:
            dW = jl_empty((M, K), W.dtype, W.device)
            dx = dx2 = jl_empty((K, N), W.dtype, W.device)
            db = jl_empty((M,), W.dtype, W.device) if bb is not None else None
        y2, pre2 = y.reshape(M, N), (None if pre is None else pre.reshape(M, N))
        _, wsp, wsn = _ws(lib.lb2_dense_bwd_workspace_bytes(M, N, K, dt, code, flags), W.device)
        _cabi.check(lib.lb2_dense_bwd(ptr(dW), ptr(dx2), ptr(db), ptr(d), None if keep_pre else ptr(y2), ptr(pre2),
                                      ptr(W), ptr(X), M, N, K, ldw, ldx, max(M, 1), dt, code, int(shadows is not None),
                                      flags, wsp, wsn, current_stream(W.device)))
        if shadows is not None:
            if delta.dtype == W.dtype:
                delta.zero_()      # dy .= 0 is the caller-side half of the contract (impl/dense.jl:281)
            return dW, dx, db
        return dW, (dx.reshape(x.shape) if x.dim() == 1 else dx), db

    return y, pullback


def matmul(A, B, *, transA=False, transB=False, flags: int = 0, out=None, accumulate=False):
    """op(A) * op(B) on column-major matrices — matmul! (lib/LuxLib/src/impl/matmul.jl:96-125).
    `out` names the destination; with `accumulate` the product is added to it (mul!(C, A, B, true, true), the form
    the Enzyme rules of matmuladd! use, lib/LuxLib/src/impl/matmul.jl:254-347)."""
    lib = _cabi.load()
    A, B = _promote(A, B)
    A2, lda = _matrix_ld(A)
    B2, ldb = _matrix_ld(B)
    M, K = (A2.shape[1], A2.shape[0]) if transA else A2.shape
    Kb, N = (B2.shape[1], B2.shape[0]) if transB else B2.shape
    if K != Kb:
        raise DimensionMismatch(f"inner dimensions differ: {K} vs {Kb}")
    dt = dtype_code(A2.dtype)
    if out is None:
        if accumulate:
            raise ArgumentError("accumulate needs the destination `out`")
        Cm, ldc = jl_empty((M, N), A2.dtype, A2.device), max(M, 1)
    else:
        if tuple(out.shape) != (M, N) or out.dtype != A2.dtype:
            raise DimensionMismatch(f"out must be a {M} x {N} matrix of {A2.dtype}")
        Cm, ldc = _matrix_ld(out)
        if Cm is not out:
            raise ArgumentError("out must be column-major with a contiguous first index")
    _, wsp, wsn = _ws(lib.lb2_matmul_workspace_bytes(M, N, K, dt, flags), A2.device)
    _cabi.check(lib.lb2_matmul(ptr(Cm), ptr(A2), ptr(B2), M, N, K, lda, ldb, ldc, int(transA), int(transB), dt,
                               int(bool(accumulate)), flags, wsp, wsn, current_stream(A2.device)))
    return Cm


# --------------------------------------------------------------------------------------------
# bias + activation
# --------------------------------------------------------------------------------------------
def _scb(x: torch.Tensor):
    """(S, C, B) view sizes of lib/LuxLib/src/impl/bias_activation.jl:229-235."""
    if x.dim() == 1:
        return 1, x.shape[0], 1
    s = 1
    for d in x.shape[:-2]:
        s *= d
    return s, x.shape[-2], x.shape[-1]


def bias_activation(act: str, x, bias=None):
    """act.(x .+ bias) with bias along dim N-1 — lib/LuxLib/src/api/bias_activation.jl:15-45."""
    lib = _cabi.load()
    x, bias = _promote(x, bias)
    S, Cc, B = _scb(x)
    if bias is not None and bias.shape[0] != Cc:
        raise DimensionMismatch("length(bias) must equal size(x, N-1)")
    X = as_colmajor(x)
    y = jl_empty(X.shape, X.dtype, X.device)
    _cabi.check(lib.lb2_bias_act_fwd(ptr(y), ptr(X), ptr(bias), S, Cc, B, dtype_code(X.dtype), act_code(act),
                                     current_stream(X.device)))
    return y


def fast_activation(act: str, x):
    """act.(x) — lib/LuxLib/src/api/activation.jl (fast_activation)."""
    return bias_activation(act, x, None)


def rrule_bias_activation(act: str, x, bias=None):
    """rrule(bias_activation) — lib/LuxLib/src/impl/bias_activation.jl:55-141."""
    lib = _cabi.load()
    x, bias = _promote(x, bias)
    S, Cc, B = _scb(x)
    X = as_colmajor(x)
    code = act_code(act)
    keep_pre = needs_preactivation(act)
    pre = bias_activation("identity", X, bias) if keep_pre else None
    y = bias_activation(act, X, bias)

    def pullback(delta):
        d = as_colmajor(delta.to(X.dtype))
        dx = jl_empty(X.shape, X.dtype, X.device)
        db = jl_empty((Cc,), X.dtype, X.device) if bias is not None else None
        _, wsp, wsn = _ws(lib.lb2_bias_act_bwd_workspace_bytes(S, Cc, B), X.device)
        _cabi.check(lib.lb2_bias_act_bwd(ptr(dx), ptr(db), ptr(d), None if keep_pre else ptr(y), ptr(pre), S, Cc, B,
                                         dtype_code(X.dtype), code, wsp, wsn, current_stream(X.device)))
        return dx, db

    return y, pullback


def rrule_scale(act: str, weight, x, bias=None):
    """The Scale layer (src/layers/basic.jl:452-461): y = act.(x .* weight .+ bias), weight / bias of the layer's dims,
    x of shape (dims..., batch...); pullback Δ -> (∂weight, ∂x, ∂bias) of the broadcast."""
    lib = _cabi.load()
    weight, x, bias = _promote(weight, x, bias)
    nd = weight.dim()
    if x.dim() < nd or tuple(x.shape[:nd]) != tuple(weight.shape):
        raise DimensionMismatch(f"x of size {tuple(x.shape)} does not start with the layer's dims {tuple(weight.shape)}")
    if bias is not None and tuple(bias.shape) != tuple(weight.shape):
        raise DimensionMismatch("weight and bias must have the same shape")
    X, Wt = as_colmajor(x), as_colmajor(weight)
    Bs = as_colmajor(bias) if bias is not None else None
    D = Wt.numel()
    B = X.numel() // D if D else 0
    code, dt = act_code(act), dtype_code(X.dtype)
    y = jl_empty(X.shape, X.dtype, X.device)
    _cabi.check(lib.lb2_scale_fwd(ptr(y), ptr(X), ptr(Wt), ptr(Bs), D, B, dt, code, current_stream(X.device)))

    def pullback(delta):
        d = as_colmajor(delta.to(X.dtype))
        dx = jl_empty(X.shape, X.dtype, X.device)
        dw = jl_empty(Wt.shape, X.dtype, X.device)
        db = jl_empty(Wt.shape, X.dtype, X.device) if Bs is not None else None
        _, wsp, wsn = _ws(lib.lb2_scale_bwd_workspace_bytes(D, B), X.device)
        _cabi.check(lib.lb2_scale_bwd(ptr(dx), ptr(dw), ptr(db), ptr(d), ptr(X), ptr(Wt), ptr(Bs), D, B, dt, code, wsp, wsn,
                                      current_stream(X.device)))
        return dw, dx, db

    return y, pullback


def scale(act: str, weight, x, bias=None):
    """act.(x .* weight .+ bias) — the Scale layer (src/layers/basic.jl:452-461)."""
    return rrule_scale(act, weight, x, bias)[0]


def _add_act(code: int, X, Y):
    lib = _cabi.load()
    z = jl_empty(X.shape, X.dtype, X.device)
    n = X.numel()
    # the bias-activation kernel with one "channel" per element: z[e] = act(x[e] + y[e])
    _cabi.check(lib.lb2_bias_act_fwd(ptr(z), ptr(X), ptr(Y), 1, n, 1, dtype_code(X.dtype), code, current_stream(X.device)))
    return z


def add_activation(act: str, x, y):
    """act.(x .+ y) for two arrays of one shape: the residual join of a ResNet block
    (perf/resnet/resnet.jl:6-7), on the bias-activation kernel."""
    if tuple(x.shape) != tuple(y.shape):
        raise DimensionMismatch("x and y must have the same shape")
    x, y = _promote(x, y)
    return _add_act(act_code(act), as_colmajor(x), as_colmajor(y))


def rrule_add_activation(act: str, x, y):
    """Forward + pullback Δ -> (∂x, ∂y) of act.(x .+ y); both inputs receive Δ .* act'."""
    if tuple(x.shape) != tuple(y.shape):
        raise DimensionMismatch("x and y must have the same shape")
    lib = _cabi.load()
    x, y = _promote(x, y)
    X, Y = as_colmajor(x), as_colmajor(y)
    code = act_code(act)
    keep_pre = needs_preactivation(act)
    pre = _add_act(_cabi.ACT_IDENTITY, X, Y) if keep_pre else None
    z = _add_act(code, X, Y)

    def pullback(delta):
        d = as_colmajor(delta.to(X.dtype))
        if code == _cabi.ACT_IDENTITY:
            return d, d
        g = jl_empty(X.shape, X.dtype, X.device)
        _cabi.check(lib.lb2_act_bwd(ptr(g), ptr(d), None if keep_pre else ptr(z), ptr(pre), X.numel(), dtype_code(X.dtype), code,
                                    current_stream(X.device)))
        return g, g

    return z, pullback


# --------------------------------------------------------------------------------------------
# convolution
# --------------------------------------------------------------------------------------------
@dataclass
class ConvDims:
    """The fields of NNlib.DenseConvDims built at src/layers/conv.jl:253-256."""
    stride: Tuple[int, ...]
    padding: Tuple[int, ...]   # (lo_1, hi_1, lo_2, hi_2, ...)
    dilation: Tuple[int, ...]
    groups: int = 1
    flipkernel: bool = False   # False: true convolution (Lux default); True: cross-correlation

    @staticmethod
    def make(nd: int, stride=1, padding=0, dilation=1, groups=1, flipkernel=False) -> "ConvDims":
        def tup(v, n):
            return tuple(int(q) for q in v) if isinstance(v, (tuple, list)) else (int(v),) * n
        s, d, p = tup(stride, nd), tup(dilation, nd), tup(padding, 2 * nd)
        if len(p) == nd:
            p = tuple(q for v in p for q in (v, v))
        if not (len(s) == nd and len(d) == nd and len(p) == 2 * nd):
            raise DimensionMismatch("stride / dilation / padding rank does not match the spatial rank")
        return ConvDims(s, p, d, int(groups), bool(flipkernel))


def _conv_desc_from(wshape, spatial, cin: int, batch: int, cd: ConvDims) -> _cabi.ConvDesc:
    """lb2_conv_desc of the convolution that maps an input of spatial extents `spatial` with `cin` channels through a
    filter of shape `wshape` = (k..., cin / groups, cout)."""
    nd = len(spatial)
    if len(wshape) != nd + 2 or nd < 1 or nd > 3:
        raise DimensionMismatch("weight and x must have the same rank (3 to 5)")
    if len(cd.stride) != nd:
        raise DimensionMismatch("ConvDims rank does not match the arrays")
    cin_g, cout = wshape[-2], wshape[-1]
    if cin_g * cd.groups != cin or cout % cd.groups != 0:
        raise DimensionMismatch(f"channels: x has {cin}, weight expects {cin_g} x {cd.groups} groups -> {cout}")
    d = _cabi.ConvDesc()
    d.ndim = nd
    for i in range(3):
        live = i < nd
        d.in_[i] = spatial[i] if live else 1
        d.k[i] = wshape[i] if live else 1
        d.stride[i] = cd.stride[i] if live else 1
        d.pad_lo[i] = cd.padding[2 * i] if live else 0
        d.pad_hi[i] = cd.padding[2 * i + 1] if live else 0
        d.dilation[i] = cd.dilation[i] if live else 1
    d.groups, d.flipkernel, d.cin, d.cout, d.batch = cd.groups, int(cd.flipkernel), cin, cout, batch
    return d


def _conv_desc(weight, x, cd: ConvDims) -> _cabi.ConvDesc:
    if weight.dim() != x.dim():
        raise DimensionMismatch("weight and x must have the same rank (3 to 5)")
    return _conv_desc_from(tuple(weight.shape), tuple(x.shape[:-2]), x.shape[-2], x.shape[-1], cd)


def _conv_fwd(act, weight, x, b, cd, want_preact, flags=0, want_ws=False):
    lib = _cabi.load()
    weight, x, b = _promote(weight, x, b)
    d = _conv_desc(weight, x, cd)
    if b is not None and b.shape[0] != d.cout:
        raise DimensionMismatch("length(bias) must equal the number of output channels")
    Wt, X = as_colmajor(weight), as_colmajor(x)
    osz = (C.c_int32 * 3)()
    _cabi.check(lib.lb2_conv_output_size(C.byref(d), osz))
    yshape = tuple(osz[i] for i in range(d.ndim)) + (d.cout, d.batch)
    y = jl_empty(yshape, X.dtype, X.device)
    pre = jl_empty(yshape, X.dtype, X.device) if want_preact else None
    dt = dtype_code(X.dtype)
    ws, wsp, wsn = _ws(lib.lb2_conv_fwd_workspace_bytes(C.byref(d), dt), X.device)
    _cabi.check(lib.lb2_conv_fwd(ptr(y), ptr(pre), ptr(X), ptr(Wt), ptr(b), C.byref(d), dt, act_code(act), flags, wsp, wsn,
                                 current_stream(X.device)))
    # the general tensor-core path leaves its channel-innermost copy of x at the start of the workspace; a pullback
    # that keeps the workspace alive hands it back instead of having the copy made again
    keep = ws if (want_ws and ws is not None and not (flags & _cabi.FLAG_FORCE_SIMT) and X.data_ptr() % 16 == 0 and
                  lib.lb2_conv_fwd_leaves_x_copy(C.byref(d), dt) == 1) else None
    return y, pre, (Wt, X, b, d, dt, keep)


def fused_conv_bias_activation(act: str, weight, x, b, cdims: ConvDims, *, flags: int = 0):
    """act.(conv(x, weight, cdims) .+ b) — lib/LuxLib/src/api/conv.jl:30-38."""
    return _conv_fwd(act, weight, x, b, cdims, False, flags)[0]


def rrule_fused_conv(act: str, weight, x, b, cdims: ConvDims, *, flags: int = 0):
    """rrule(fused_conv) + ∇fused_conv — lib/LuxLib/src/impl/conv.jl:204-275.
    Pullback Δ -> (∂weight, ∂x, ∂b)."""
    lib = _cabi.load()
    keep_pre = needs_preactivation(act)
    y, pre, (Wt, X, bb, d, dt, xcopy) = _conv_fwd(act, weight, x, b, cdims, keep_pre, flags, want_ws=True)
    code = act_code(act)

    def pullback(delta, need_dx=True):
        """Δ -> (∂weight, ∂x, ∂b); `need_dx=False` (a network's first layer) skips the data gradient and returns None for it."""
        dl = as_colmajor(delta.to(X.dtype))  # NNlib.colmajor(Δ): impl/conv.jl:263
        dw = jl_empty(Wt.shape, X.dtype, X.device)
        dx = jl_empty(X.shape, X.dtype, X.device) if need_dx else None
        db = jl_empty((d.cout,), X.dtype, X.device) if bb is not None else None
        _, wsp, wsn = _ws(lib.lb2_conv_bwd_workspace_bytes(C.byref(d), dt, code), X.device)
        xarg, xflag = (ptr(xcopy), _cabi.FLAG_X_COPY_GIVEN) if xcopy is not None else (ptr(X), 0)
        _cabi.check(lib.lb2_conv_bwd(ptr(dw), ptr(dx), ptr(db), ptr(dl), None if keep_pre else ptr(y), ptr(pre), xarg,
                                     ptr(Wt), C.byref(d), dt, code, flags | xflag, wsp, wsn, current_stream(X.device)))
        return dw, dx, db

    return y, pullback


def conv_transpose_output_size(in_sz, k, cd: ConvDims, outpad=0):
    """Spatial size of conv_transpose's result (conv_transpose_dims, src/layers/conv.jl:19-45): the input size of the
    convolution whose output has size `in_sz`: (in - 1)*stride + 1 + (k - 1)*dilation - pad_lo - pad_hi + outpad."""
    nd = len(in_sz)
    op = tuple(outpad) if isinstance(outpad, (tuple, list)) else (int(outpad),) * nd
    return tuple((in_sz[i] - 1) * cd.stride[i] + 1 + (k[i] - 1) * cd.dilation[i] - cd.padding[2 * i] - cd.padding[2 * i + 1] + op[i]
                 for i in range(nd))


def rrule_conv_transpose(act: str, weight, x, b, cdims: ConvDims, outpad=0, *, flags: int = 0):
    """The ConvTranspose layer's computation (src/layers/conv.jl:428-434): act.(conv_transpose(x, weight, cdims) .+ b) with
    NNlib.conv_transpose(x, w, cdims) = ∇conv_data(x, w, cdims), and its pullback Δ -> (∂weight, ∂x, ∂b). `weight` is
    (k..., C_out / groups, C_in) — the filter of the convolution that maps the RESULT back onto x. Everything runs on the
    convolution entry points: forward = the data-gradient kernels + the bias-activation kernel; pullback: ∂x = conv(g, w),
    ∂weight = ∇conv_filter(g, x) with g = Δ .* act'."""
    lib = _cabi.load()
    weight, x, b = _promote(weight, x, b)
    if weight.dim() != x.dim():
        raise DimensionMismatch("weight and x must have the same rank (3 to 5)")
    Wt, X = as_colmajor(weight), as_colmajor(x)
    nd = X.dim() - 2
    if Wt.shape[-1] != X.shape[-2]:
        raise DimensionMismatch(f"x has {X.shape[-2]} channels, weight expects {Wt.shape[-1]}")
    cu = Wt.shape[-2] * cdims.groups
    usz = conv_transpose_output_size(tuple(X.shape[:nd]), tuple(Wt.shape[:nd]), cdims, outpad)
    d = _conv_desc_from(tuple(Wt.shape), usz, cu, X.shape[-1], cdims)
    osz = (C.c_int32 * 3)()
    _cabi.check(lib.lb2_conv_output_size(C.byref(d), osz))
    if tuple(osz[i] for i in range(nd)) != tuple(X.shape[:nd]):
        raise DimensionMismatch("outpad does not fit the stride: the convolution of the result does not reproduce size(x)")
    if b is not None and b.shape[0] != cu:
        raise DimensionMismatch("length(bias) must equal the number of output channels")
    dt = dtype_code(X.dtype)
    ident = act_code("identity")
    u = jl_empty(usz + (cu, X.shape[-1]), X.dtype, X.device)
    _, wsp, wsn = _ws(lib.lb2_conv_bwd_workspace_bytes(C.byref(d), dt, ident), X.device)
    _cabi.check(lib.lb2_conv_bwd(None, ptr(u), None, ptr(X), None, None, None, ptr(Wt), C.byref(d), dt, ident, flags, wsp, wsn,
                                 current_stream(X.device)))
    y, pb_act = rrule_bias_activation(act, u, b)

    def pullback(delta):
        g, db = pb_act(delta)
        dx = jl_empty(X.shape, X.dtype, X.device)
        _, w1, n1 = _ws(lib.lb2_conv_fwd_workspace_bytes(C.byref(d), dt), X.device)
        _cabi.check(lib.lb2_conv_fwd(ptr(dx), None, ptr(g), ptr(Wt), None, C.byref(d), dt, ident, flags, w1, n1, current_stream(X.device)))
        dw = jl_empty(Wt.shape, X.dtype, X.device)
        _, w2, n2 = _ws(lib.lb2_conv_bwd_workspace_bytes(C.byref(d), dt, ident), X.device)
        _cabi.check(lib.lb2_conv_bwd(ptr(dw), None, None, ptr(X), None, None, ptr(g), None, C.byref(d), dt, ident, flags, w2, n2,
                                     current_stream(X.device)))
        return dw, dx, db

    return y, pullback


def conv_transpose_bias_activation(act: str, weight, x, b, cdims: ConvDims, outpad=0, *, flags: int = 0):
    """act.(conv_transpose(x, weight, cdims) .+ b) — the ConvTranspose layer (src/layers/conv.jl:428-434)."""
    return rrule_conv_transpose(act, weight, x, b, cdims, outpad, flags=flags)[0]


# --------------------------------------------------------------------------------------------
# batched matrix product, attention
# --------------------------------------------------------------------------------------------
def _bmm(lib, Cp, Ap, Bp, M, N, K, batch, lda, ldb, ldc, sa, sb, sc, ta, tb, dt, device, accumulate=0, flags=0):
    """One lb2_batched_matmul call on raw pointers (integers)."""
    _, wsp, wsn = _ws(lib.lb2_batched_matmul_workspace_bytes(M, N, K, dt, flags), device)
    _cabi.check(lib.lb2_batched_matmul(Cp, Ap, Bp, M, N, K, batch, lda, ldb, ldc, sa, sb, sc, int(ta), int(tb), dt, accumulate, flags,
                                       wsp, wsn, current_stream(device)))


def batched_matmul(x, y, *, flags: int = 0):
    """LuxLib.batched_matmul(x, y) (lib/LuxLib/src/api/batched_mul.jl:56-70) for the default dimension roles:
    x (M, K, Bx), y (K, N, By) -> (M, N, max(Bx, By)); a matrix counts as batch size 1 and a batch dimension of size 1
    is repeated. Batch dimensions beyond the third are flattened like the reference does."""
    lib = _cabi.load()
    x, y = _promote(x, y)
    if x.dim() == 2:
        x = jl_reshape(x, (x.shape[0], x.shape[1], 1))
    if y.dim() == 2:
        y = jl_reshape(y, (y.shape[0], y.shape[1], 1))
    if x.dim() != y.dim() or x.dim() < 3:
        raise DimensionMismatch("batched_matmul needs two arrays of the same rank (>= 3) or a matrix and a 3-D array")
    X, Y = as_colmajor(x), as_colmajor(y)
    bx, by = tuple(X.shape[2:]), tuple(Y.shape[2:])
    if any(p != q and p != 1 and q != 1 for p, q in zip(bx, by)):
        raise DimensionMismatch(f"batch dimensions {bx} and {by} do not match")
    if len(bx) > 1 and bx != by:      # mixed repeats over several batch dimensions: materialise them like Utils.maybe_repeat
        full = tuple(max(p, q) for p, q in zip(bx, by))
        X = as_colmajor(X.expand(*X.shape[:2], *full))
        Y = as_colmajor(Y.expand(*Y.shape[:2], *full))
        bx = by = full
    M, K = X.shape[0], X.shape[1]
    if Y.shape[0] != K:
        raise DimensionMismatch(f"size(x, 2) = {K} does not match size(y, 1) = {Y.shape[0]}")
    N = Y.shape[1]
    nbx, nby = math.prod(bx), math.prod(by)
    nb = max(nbx, nby)
    out = jl_empty((M, N) + tuple(max(p, q) for p, q in zip(bx, by)), X.dtype, X.device)
    _bmm(lib, ptr(out), ptr(X), ptr(Y), M, N, K, nb, max(M, 1), max(K, 1), max(M, 1), 0 if nbx == 1 else M * K, 0 if nby == 1 else K * N,
         M * N, 0, 0, dtype_code(X.dtype), X.device, flags=flags)
    return out


def rrule_batched_matmul(x, y, *, flags: int = 0):
    """batched_matmul with its pullback Δ -> (∂x, ∂y): ∂x = Δ ⊠ yᵀ, ∂y = xᵀ ⊠ Δ (summed over a repeated batch)."""
    lib = _cabi.load()
    z = batched_matmul(x, y, flags=flags)
    x, y = _promote(x, y)
    X3 = jl_reshape(x, (x.shape[0], x.shape[1], math.prod(x.shape[2:])))
    Y3 = jl_reshape(y, (y.shape[0], y.shape[1], math.prod(y.shape[2:])))
    M, K, nbx = X3.shape
    N, nby = Y3.shape[1], Y3.shape[2]
    nb = max(nbx, nby)
    if x.dim() > 3 and tuple(x.shape[2:]) != tuple(y.shape[2:]):
        raise NotImplementedError("pullback with mixed repeats over several batch dimensions")
    dt, es = dtype_code(X3.dtype), X3.element_size()

    def pullback(delta):
        D = as_colmajor(delta.to(X3.dtype))
        dx = jl_empty(tuple(x.shape), X3.dtype, X3.device)
        dy = jl_empty(tuple(y.shape), X3.dtype, X3.device)
        # a repeated operand's gradient is the sum over the batch: accumulate element by element in a fixed order
        if nbx == nb:
            _bmm(lib, ptr(dx), ptr(D), ptr(Y3), M, K, N, nb, M, K, M, M * N, 0 if nby == 1 else K * N, M * K, 0, 1, dt, X3.device, flags=flags)
        else:
            for i in range(nb):
                _bmm(lib, ptr(dx), D.data_ptr() + i * M * N * es, Y3.data_ptr() + (0 if nby == 1 else i * K * N * es), M, K, N, 1, M, K, M,
                     0, 0, M * K, 0, 1, dt, X3.device, accumulate=1 if i else 0, flags=flags)
        if nby == nb:
            _bmm(lib, ptr(dy), ptr(X3), ptr(D), K, N, M, nb, M, M, K, 0 if nbx == 1 else M * K, M * N, K * N, 1, 0, dt, X3.device, flags=flags)
        else:
            for i in range(nb):
                _bmm(lib, ptr(dy), X3.data_ptr() + (0 if nbx == 1 else i * M * K * es), D.data_ptr() + i * M * N * es, K, N, M, 1, M, M, K,
                     0, 0, K * N, 1, 0, dt, X3.device, accumulate=1 if i else 0, flags=flags)
        return dx, dy

    return z, pullback


def rrule_scaled_dot_product_attention(q, k, v, *, scale=None, mask=None, is_causal=None, bias=None, flags: int = 0):
    """LuxLib.scaled_dot_product_attention (lib/LuxLib/src/api/attention.jl, impl/attention.jl:5-118) for the default
    dimension roles head_dim = 1, token_dim = 3: q (D, H, L, B...), k (D, Hkv, S, B...), v (E, Hkv, S, B...) ->
    (x (E, H, L, B...), weights (S, L, H, B...)), and the pullback (Δx) -> (∂q, ∂k, ∂v, ∂bias). Logits =
    batched k'q / scale (default scale sqrt(D)), + bias, masked (mask true = keep, or is_causal), softmax over the key
    index. H must be a multiple of Hkv (grouped keys / values are shared by consecutive query heads)."""
    lib = _cabi.load()
    if q.dim() < 4 or k.dim() != q.dim() or v.dim() != q.dim():
        raise AssertionError("N must be at least 4")
    if mask is not None and is_causal is not None:
        raise AssertionError("`mask` and `is_causal` cannot both be specified")
    q, k, v = _promote(q, k, v)
    Q, Kx, V = as_colmajor(q), as_colmajor(k), as_colmajor(v)
    D, H, Lq = Q.shape[:3]
    Hkv, S = Kx.shape[1], Kx.shape[2]
    E = V.shape[0]
    if Kx.shape[0] != D:
        raise AssertionError("`q` and `k` must have the same head dimension")
    if tuple(Q.shape[3:]) != tuple(Kx.shape[3:]) or tuple(Q.shape[3:]) != tuple(V.shape[3:]):
        raise DimensionMismatch("All dimensions (except first 3) of q, k, v must be the same")
    if V.shape[2] != S or V.shape[1] != Hkv:
        raise AssertionError("`v` and `k` must have the same number of tokens and heads")
    if H % Hkv != 0:
        raise AssertionError("num_heads must be divisible by num_kv_groups")
    gs = H // Hkv
    batch_shape = tuple(Q.shape[3:])
    Bn = math.prod(batch_shape)
    sc = 1.0 / (float(scale) if scale is not None else float(D) ** 0.5)
    dt, es, device = dtype_code(Q.dtype), Q.element_size(), Q.device
    logits = jl_empty((S, Lq, H) + batch_shape, Q.dtype, device)

    def per_group(fn):
        for b in range(Bn):
            for g in range(Hkv):
                fn(b, g)

    # logits[:, :, h, b] = k[:, g, :, b]' * q[:, h, :, b] for the gs heads h of group g: one batched call, k repeated
    def fwd_logits(b, g):
        _bmm(lib, logits.data_ptr() + ((g * gs + H * b) * S * Lq) * es, Kx.data_ptr() + (g * D + b * D * Hkv * S) * es,
             Q.data_ptr() + (g * gs * D + b * D * H * Lq) * es, S, Lq, D, gs, D * Hkv, D * H, S, 0, D, S * Lq, 1, 0, dt, device, flags=flags)
    per_group(fwd_logits)

    bias_c = mask_c = None
    bias_bs = mask_bs = 0
    if bias is not None:
        bias_c = as_colmajor(bias.to(Q.dtype))
        if tuple(bias_c.shape) == (S, Lq):
            bias_bs = 0
        elif tuple(bias_c.shape) == (S, Lq, H) + batch_shape:
            bias_bs = S * Lq
        else:
            raise DimensionMismatch("bias must have the shape (S, L) or (S, L, H, B...)")
    if mask is not None:
        mask_c = as_colmajor(mask.to(torch.uint8))
        if tuple(mask_c.shape) == (S, Lq):
            mask_bs = 0
        elif tuple(mask_c.shape) == (S, Lq, H) + batch_shape:
            mask_bs = S * Lq
        else:
            raise DimensionMismatch("mask must have the shape (S, L) or (S, L, H, B...)")
    w = jl_empty(tuple(logits.shape), Q.dtype, device)
    _cabi.check(lib.lb2_attention_softmax_fwd(ptr(w), ptr(logits), ptr(bias_c), bias_bs, ptr(mask_c), mask_bs, 1 if is_causal else 0, sc,
                                              S, Lq, H * Bn, dt, current_stream(device)))
    out = jl_empty((E, H, Lq) + batch_shape, Q.dtype, device)

    # x[:, h, :, b] = v[:, g, :, b] * w[:, :, h, b]
    def fwd_out(b, g):
        _bmm(lib, out.data_ptr() + (g * gs * E + b * E * H * Lq) * es, V.data_ptr() + (g * E + b * E * Hkv * S) * es,
             w.data_ptr() + ((g * gs + H * b) * S * Lq) * es, E, Lq, S, gs, E * Hkv, S, E * H, 0, S * Lq, E, 0, 0, dt, device, flags=flags)
    per_group(fwd_out)

    def pullback(dx):
        G = as_colmajor(dx.to(Q.dtype))
        dw = jl_empty(tuple(w.shape), Q.dtype, device)
        dq, dk, dv = (jl_empty(tuple(t.shape), Q.dtype, device) for t in (Q, Kx, V))

        # dw[:, :, h, b] = v[:, g, :, b]' * dx[:, h, :, b]
        def bwd_dw(b, g):
            _bmm(lib, dw.data_ptr() + ((g * gs + H * b) * S * Lq) * es, V.data_ptr() + (g * E + b * E * Hkv * S) * es,
                 G.data_ptr() + (g * gs * E + b * E * H * Lq) * es, S, Lq, E, gs, E * Hkv, E * H, S, 0, E, S * Lq, 1, 0, dt, device, flags=flags)
        per_group(bwd_dw)
        dl = jl_empty(tuple(w.shape), Q.dtype, device)
        db = jl_empty(tuple(w.shape), Q.dtype, device) if bias_c is not None else None
        _cabi.check(lib.lb2_attention_softmax_bwd(ptr(dl), ptr(db), ptr(dw), ptr(w), sc, S, Lq, H * Bn, dt, current_stream(device)))

        # per head (the heads of a group add into the same dk / dv, so they run one after the other, in order):
        # dv[:, g, :, b] += dx[:, h, :, b] * w[:, :, h, b]';  dk[:, g, :, b] += q[:, h, :, b] * dl[:, :, h, b]'
        # dq[:, h, :, b] = k[:, g, :, b] * dl[:, :, h, b]
        def bwd_rest(b, g):
            _bmm(lib, dq.data_ptr() + (g * gs * D + b * D * H * Lq) * es, Kx.data_ptr() + (g * D + b * D * Hkv * S) * es,
                 dl.data_ptr() + ((g * gs + H * b) * S * Lq) * es, D, Lq, S, gs, D * Hkv, S, D * H, 0, S * Lq, D, 0, 0, dt, device, flags=flags)
            for j in range(gs):
                h = g * gs + j
                _bmm(lib, dv.data_ptr() + (g * E + b * E * Hkv * S) * es, G.data_ptr() + (h * E + b * E * H * Lq) * es,
                     w.data_ptr() + ((h + H * b) * S * Lq) * es, E, S, Lq, 1, E * H, S, E * Hkv, 0, 0, E * S, 0, 1, dt, device,
                     accumulate=1 if j else 0, flags=flags)
                _bmm(lib, dk.data_ptr() + (g * D + b * D * Hkv * S) * es, Q.data_ptr() + (h * D + b * D * H * Lq) * es,
                     dl.data_ptr() + ((h + H * b) * S * Lq) * es, D, S, Lq, 1, D * H, S, D * Hkv, 0, 0, D * S, 0, 1, dt, device,
                     accumulate=1 if j else 0, flags=flags)
        per_group(bwd_rest)
        if db is not None and bias_bs == 0:
            # a bias shared by all heads and samples: its gradient is the sum over them — the bias-gradient reduction on
            # the (1, S*L, H*B) view
            full, db = db, jl_empty((S, Lq), Q.dtype, device)
            _, wsp, wsn = _ws(lib.lb2_bias_act_bwd_workspace_bytes(1, S * Lq, H * Bn), device)
            _cabi.check(lib.lb2_bias_act_bwd(None, ptr(db), ptr(full), None, None, 1, S * Lq, H * Bn, dt, act_code("identity"), wsp, wsn,
                                             current_stream(device)))
        return dq, dk, dv, db

    return (out, w), pullback


def scaled_dot_product_attention(q, k, v, **kw):
    """(x, attention weights) of LuxLib.scaled_dot_product_attention for head_dim = 1, token_dim = 3."""
    return rrule_scaled_dot_product_attention(q, k, v, **kw)[0]


# --------------------------------------------------------------------------------------------
# normalisation
# --------------------------------------------------------------------------------------------
def default_epsilon(dtype: torch.dtype) -> float:
    """eps(T)^(5/7) — lib/LuxLib/src/utils.jl:130."""
    return float(torch.finfo(dtype).eps) ** (5.0 / 7.0)


def _check_affine(scale, bias):
    if (scale is None) != (bias is None):
        raise ArgumentError("scale and bias must both be given or both be nothing")


def batchnorm(x, scale, bias, running_mean, running_var, training: bool, act: str = "identity",
              momentum: float = 0.1, epsilon: Optional[float] = None):
    """LuxLib.batchnorm — lib/LuxLib/src/api/batchnorm.jl:31-55.

    Returns (y, (running_mean′, running_var′)). The four statistics cases of
    lib/LuxLib/src/impl/normalization.jl:116-143 apply: training with running statistics updates
    them (new arrays); training without returns (None, None); inference with running statistics
    uses them unchanged; inference without falls back to batch statistics."""
    y, stats, _ = _batchnorm_fwd(x, scale, bias, running_mean, running_var, training, act, momentum, epsilon)
    return y, stats


def _batchnorm_fwd(x, scale, bias, rmean, rvar, training, act, momentum, epsilon):
    lib = _cabi.load()
    _check_affine(scale, bias)
    if (rmean is None) != (rvar is None):
        raise ArgumentError("running_mean and running_var must both be given or both be nothing")
    if x.dim() < 2:
        raise DimensionMismatch("batchnorm needs at least 2 dims (channels, batch)")
    X = as_colmajor(x)
    S, Cc, B = _scb(X)
    for v, name in ((scale, "scale"), (bias, "bias"), (rmean, "running_mean"), (rvar, "running_var")):
        if v is not None and v.shape[0] != Cc:
            raise DimensionMismatch(f"length({name}) must equal the number of channels {Cc}")
    eps = default_epsilon(X.dtype) if epsilon is None else float(epsilon)
    dt = dtype_code(X.dtype)
    dev = X.device
    y = jl_empty(X.shape, X.dtype, dev)
    code = act_code(act)
    cast = lambda v: None if v is None else v.to(X.dtype)
    scale_c, bias_c, rmean_c, rvar_c = cast(scale), cast(bias), cast(rmean), cast(rvar)
    if training or rmean is None:
        save_mean = torch.empty(Cc, dtype=torch.float32, device=dev)
        save_inv = torch.empty(Cc, dtype=torch.float32, device=dev)
        update = training and rmean is not None
        new_rm = torch.empty_like(rmean_c) if update else None
        new_rv = torch.empty_like(rvar_c) if update else None
        _, wsp, wsn = _ws(lib.lb2_batchnorm_workspace_bytes(S, Cc, B), dev)
        _cabi.check(lib.lb2_batchnorm_fwd_train(ptr(y), ptr(save_mean), ptr(save_inv), ptr(new_rm), ptr(new_rv), ptr(X),
                                                ptr(scale_c), ptr(bias_c), ptr(rmean_c) if update else None,
                                                ptr(rvar_c) if update else None, S, Cc, B, float(momentum), eps, dt,
                                                code, wsp, wsn, current_stream(dev)))
        stats = (new_rm, new_rv) if update else (rmean, rvar)
        return y, stats, (X, scale_c, bias_c, save_mean, save_inv, S, Cc, B, dt, code, True)
    _cabi.check(lib.lb2_batchnorm_fwd_infer(ptr(y), ptr(X), ptr(scale_c), ptr(bias_c), ptr(rmean_c), ptr(rvar_c), S, Cc, B,
                                            eps, dt, code, current_stream(dev)))
    return y, (rmean, rvar), (X, scale_c, bias_c, (rmean_c, eps), rvar_c, S, Cc, B, dt, code, False)


def rrule_batchnorm(x, scale, bias, running_mean, running_var, training: bool, act: str = "identity",
                    momentum: float = 0.1, epsilon: Optional[float] = None):
    """Forward + pullback Δ -> (∂x, ∂scale, ∂bias) of batchnorm:
    rrule(batchnorm_affine_normalize_internal) (lib/LuxLib/src/impl/batchnorm.jl:405-443), chained through the
    mean_var rule (lib/LuxLib/src/impl/common_ops.jl:45-61) when the statistics came from the batch. With
    training = False and running statistics given (a frozen BatchNorm being fine-tuned around) the statistics are
    constants and only the affine-normalise step is differentiated, as the reference's rule does."""
    lib = _cabi.load()
    y, stats, (X, sc, bi, save_mean, save_inv, S, Cc, B, dt, code, batch_stats) = _batchnorm_fwd(
        x, scale, bias, running_mean, running_var, training, act, momentum, epsilon)

    def pullback(delta):
        d = as_colmajor(delta.to(X.dtype))
        dx = jl_empty(X.shape, X.dtype, X.device)
        dg = torch.empty(Cc, dtype=X.dtype, device=X.device) if sc is not None else None
        db = torch.empty(Cc, dtype=X.dtype, device=X.device) if sc is not None else None
        _, wsp, wsn = _ws(lib.lb2_batchnorm_workspace_bytes(S, Cc, B), X.device)
        if batch_stats:
            _cabi.check(lib.lb2_batchnorm_bwd(ptr(dx), ptr(dg), ptr(db), ptr(d), ptr(X), ptr(sc), ptr(bi), ptr(save_mean),
                                              ptr(save_inv), S, Cc, B, dt, code, wsp, wsn, current_stream(X.device)))
        else:
            (rm, eps), rv = save_mean, save_inv
            _cabi.check(lib.lb2_batchnorm_bwd_infer(ptr(dx), ptr(dg), ptr(db), ptr(d), ptr(X), ptr(sc), ptr(bi), ptr(rm), ptr(rv),
                                                    S, Cc, B, eps, dt, code, wsp, wsn, current_stream(X.device)))
        return dx, dg, db

    return y, stats, pullback


def rrule_conv_batchnorm(act: str, weight, x, cdims: ConvDims, scale, bias, running_mean, running_var, momentum: float = 0.1,
                         epsilon: Optional[float] = None, *, flags: int = 0):
    """A bias-free Conv followed by a training-mode BatchNorm carrying the activation — the pair every block of the
    reference's ResNet is made of (perf/resnet/resnet.jl:17-22: conv_norm = Chain(Conv(...; use_bias = false),
    BatchNorm(out, act))) — with BatchNorm's statistics taken from per-channel sums that the convolution's epilogue
    forms while it writes its result, instead of a pass that reads the result back. Same values as
    batchnorm(fused_conv_bias_activation(identity, weight, x, nothing, cdims), ...) up to the summation order.
    Returns (y, (new_running_mean, new_running_var), pullback) with pullback Δ -> (∂weight, ∂x, ∂scale, ∂bias); the
    pullback is the composition of the two layers' pullbacks."""
    lib = _cabi.load()
    weight, x = _promote(weight, x)
    _check_affine(scale, bias)
    if (running_mean is None) != (running_var is None):
        raise ArgumentError("running_mean and running_var must both be given or both be nothing")
    d = _conv_desc(weight, x, cdims)
    Wt, X = as_colmajor(weight), as_colmajor(x)
    osz = (C.c_int32 * 3)()
    _cabi.check(lib.lb2_conv_output_size(C.byref(d), osz))
    ushape = tuple(osz[i] for i in range(d.ndim)) + (d.cout, d.batch)
    for v, name in ((scale, "scale"), (bias, "bias"), (running_mean, "running_mean"), (running_var, "running_var")):
        if v is not None and v.shape[0] != d.cout:
            raise DimensionMismatch(f"length({name}) must equal the number of channels {d.cout}")
    dt, dev = dtype_code(X.dtype), X.device
    if (flags & _cabi.FLAG_FORCE_SIMT) or lib.lb2_conv_fwd_sums_is_fused(C.byref(d), dt) != 1:
        # short contractions and the paths without the epilogue sums: the plain pair is the faster form
        u, pb_conv = rrule_fused_conv("identity", weight, x, None, cdims, flags=flags)
        y, stats, pb_bn = rrule_batchnorm(u, scale, bias, running_mean, running_var, True, act, momentum, epsilon)

        def pullback_pair(delta, need_dx=True):
            du, dg, db = pb_bn(delta)
            dw, dx, _ = pb_conv(du, need_dx=need_dx)
            return dw, dx, dg, db

        return y, stats, pullback_pair
    u = jl_empty(ushape, X.dtype, dev)
    sums = torch.empty(2 * d.cout, dtype=torch.float32, device=dev)
    ws, wsp, wsn = _ws(lib.lb2_conv_fwd_sums_workspace_bytes(C.byref(d), dt), dev)
    _cabi.check(lib.lb2_conv_fwd_sums(ptr(u), ptr(sums), ptr(X), ptr(Wt), C.byref(d), dt, flags, wsp, wsn, current_stream(dev)))
    xcopy = ws if (ws is not None and not (flags & _cabi.FLAG_FORCE_SIMT) and X.data_ptr() % 16 == 0 and
                   lib.lb2_conv_fwd_leaves_x_copy(C.byref(d), dt) == 1) else None
    S, Cc, B = _scb(u)
    eps = default_epsilon(X.dtype) if epsilon is None else float(epsilon)
    code = act_code(act)
    cast = lambda v: None if v is None else v.to(X.dtype)
    sc, bi, rm, rv = cast(scale), cast(bias), cast(running_mean), cast(running_var)
    y = jl_empty(ushape, X.dtype, dev)
    save_mean = torch.empty(Cc, dtype=torch.float32, device=dev)
    save_inv = torch.empty(Cc, dtype=torch.float32, device=dev)
    new_rm = torch.empty_like(rm) if rm is not None else None
    new_rv = torch.empty_like(rv) if rv is not None else None
    _, w2, n2 = _ws(lib.lb2_batchnorm_workspace_bytes(S, Cc, B), dev)
    _cabi.check(lib.lb2_batchnorm_fwd_train_sums(ptr(y), ptr(save_mean), ptr(save_inv), ptr(new_rm), ptr(new_rv), ptr(u), ptr(sc), ptr(bi),
                                                 ptr(rm), ptr(rv), ptr(sums), S, Cc, B, float(momentum), eps, dt, code, w2, n2,
                                                 current_stream(dev)))
    ident = act_code("identity")

    def pullback(delta, need_dx=True):
        dl = as_colmajor(delta.to(X.dtype))
        du = jl_empty(ushape, X.dtype, dev)
        dg = torch.empty(Cc, dtype=X.dtype, device=dev) if sc is not None else None
        db = torch.empty(Cc, dtype=X.dtype, device=dev) if sc is not None else None
        _, w3, n3 = _ws(lib.lb2_batchnorm_workspace_bytes(S, Cc, B), dev)
        _cabi.check(lib.lb2_batchnorm_bwd(ptr(du), ptr(dg), ptr(db), ptr(dl), ptr(u), ptr(sc), ptr(bi), ptr(save_mean), ptr(save_inv),
                                          S, Cc, B, dt, code, w3, n3, current_stream(dev)))
        dw = jl_empty(Wt.shape, X.dtype, dev)
        dx = jl_empty(X.shape, X.dtype, dev) if need_dx else None
        _, w4, n4 = _ws(lib.lb2_conv_bwd_workspace_bytes(C.byref(d), dt, ident), dev)
        xarg, xflag = (ptr(xcopy), _cabi.FLAG_X_COPY_GIVEN) if xcopy is not None else (ptr(X), 0)
        _cabi.check(lib.lb2_conv_bwd(ptr(dw), ptr(dx), None, ptr(du), None, None, xarg, ptr(Wt), C.byref(d), dt, ident, flags | xflag,
                                     w4, n4, current_stream(dev)))
        return dw, dx, dg, db

    return y, ((new_rm, new_rv) if rm is not None else (running_mean, running_var)), pullback


@dataclass(frozen=True)
class PoolDims:
    """The fields of NNlib.PoolDims built by calculate_pool_dims (src/layers/pooling.jl:17-34)."""
    kernel: Tuple[int, ...]
    stride: Tuple[int, ...]
    padding: Tuple[int, ...]   # (lo_1, hi_1, lo_2, hi_2, ...)
    dilation: Tuple[int, ...]

    @staticmethod
    def make(kernel, stride=None, padding=0, dilation=1) -> "PoolDims":
        k = tuple(int(q) for q in kernel) if isinstance(kernel, (tuple, list)) else (int(kernel),)
        nd = len(k)

        def tup(v, n):
            return tuple(int(q) for q in v) if isinstance(v, (tuple, list)) else (int(v),) * n
        s = k if stride is None else tup(stride, nd)   # NNlib: stride defaults to the window
        d, p = tup(dilation, nd), tup(padding, 2 * nd)
        if len(p) == nd:
            p = tuple(q for v in p for q in (v, v))
        if not (len(s) == nd and len(d) == nd and len(p) == 2 * nd):
            raise DimensionMismatch("stride / dilation / padding rank does not match the window rank")
        return PoolDims(k, s, p, d)

    @staticmethod
    def global_(x) -> "PoolDims":
        """GlobalPoolMode (src/layers/pooling.jl:21-23): the window is the whole spatial extent."""
        return PoolDims.make(tuple(x.shape[:-2]))

    @staticmethod
    def adaptive(x, out_size) -> "PoolDims":
        """AdaptivePoolMode (src/layers/pooling.jl:29-34)."""
        in_size = tuple(x.shape[:-2])
        stride = tuple(i // o for i, o in zip(in_size, out_size))
        kernel = tuple(i - (o - 1) * s for i, o, s in zip(in_size, out_size, stride))
        return PoolDims.make(kernel, stride, 0, 1)


def _pool_desc(x, pd: PoolDims) -> _cabi.PoolDesc:
    nd = x.dim() - 2
    if nd < 1 or nd > 3 or len(pd.kernel) != nd:
        raise DimensionMismatch("PoolDims rank does not match the array (3 to 5 dims: spatial..., channels, batch)")
    d = _cabi.PoolDesc()
    d.ndim = nd
    for i in range(3):
        live = i < nd
        d.in_[i] = x.shape[i] if live else 1
        d.k[i] = pd.kernel[i] if live else 1
        d.stride[i] = pd.stride[i] if live else 1
        d.pad_lo[i] = pd.padding[2 * i] if live else 0
        d.pad_hi[i] = pd.padding[2 * i + 1] if live else 0
        d.dilation[i] = pd.dilation[i] if live else 1
    d.channels, d.batch = x.shape[-2], x.shape[-1]
    return d


def _pool(kind: int, x, pd: PoolDims):
    lib = _cabi.load()
    X = as_colmajor(x)
    d = _pool_desc(X, pd)
    osz = (C.c_int32 * 3)()
    _cabi.check(lib.lb2_pool_output_size(C.byref(d), osz))
    y = jl_empty(tuple(osz[i] for i in range(d.ndim)) + (d.channels, d.batch), X.dtype, X.device)
    dt = dtype_code(X.dtype)
    _cabi.check(lib.lb2_pool_fwd(ptr(y), ptr(X), C.byref(d), kind, dt, current_stream(X.device)))

    def pullback(delta):
        dy = as_colmajor(delta.to(X.dtype))
        if tuple(dy.shape) != tuple(y.shape):
            raise DimensionMismatch("the cotangent must have the shape of the pooled output")
        dx = jl_empty(X.shape, X.dtype, X.device)
        _cabi.check(lib.lb2_pool_bwd(ptr(dx), ptr(dy), ptr(y), ptr(X), C.byref(d), kind, dt, current_stream(X.device)))
        return dx

    return y, pullback


def maxpool(x, pd: PoolDims):
    """NNlib.maxpool(x, pdims) as called by MaxPoolOp (src/layers/pooling.jl:44-46)."""
    return _pool(_cabi.POOL_MAX, x, pd)[0]


def meanpool(x, pd: PoolDims):
    """NNlib.meanpool(x, pdims) as called by MeanPoolOp (src/layers/pooling.jl:53-55)."""
    return _pool(_cabi.POOL_MEAN, x, pd)[0]


def rrule_maxpool(x, pd: PoolDims):
    """Forward + pullback Δ -> ∂x (NNlib.∇maxpool: the first maximal element of each window takes the gradient)."""
    return _pool(_cabi.POOL_MAX, x, pd)


def rrule_meanpool(x, pd: PoolDims):
    """Forward + pullback Δ -> ∂x (NNlib.∇meanpool)."""
    return _pool(_cabi.POOL_MEAN, x, pd)


def instancenorm(x, scale, bias, running_mean=None, running_var=None, training: bool = True, act: str = "identity",
                 momentum: float = 0.1, epsilon: Optional[float] = None):
    """LuxLib.instancenorm — lib/LuxLib/src/api/instancenorm.jl:32-77. Returns y, (running_mean', running_var').
    Per-instance statistics run on the groupnorm kernels with one channel per group; test mode with running
    statistics is the batchnorm inference kernel; the running-statistics update of training mode
    (lib/LuxLib/src/impl/normalization.jl:95-110) is lb2_instancenorm_update_stats."""
    if x.dim() <= 2:
        raise AssertionError(f"`ndims(x) = {x.dim()}` must be at least > 2.")
    if (running_mean is None) != (running_var is None):
        raise ArgumentError("running_mean and running_var must both be given or both be nothing")
    if running_mean is not None and not training:
        y, _ = batchnorm(x, scale, bias, running_mean, running_var, False, act, momentum, epsilon)
        return y, (running_mean, running_var)
    lib = _cabi.load()
    Cc = x.shape[-2]
    y, (X, sc, bi, sm, si, S, Cc, B, dt, code) = _groupnorm_fwd(x, scale, bias, Cc, act, epsilon)
    if running_mean is None:
        return y, (None, None)
    if running_mean.shape[0] != Cc or running_var.shape[0] != Cc:
        raise DimensionMismatch(f"length(running_mean) must equal the number of channels {Cc}")
    eps = default_epsilon(X.dtype) if epsilon is None else float(epsilon)
    rm, rv = running_mean.to(X.dtype), running_var.to(X.dtype)
    nrm, nrv = torch.empty_like(rm), torch.empty_like(rv)
    _cabi.check(lib.lb2_instancenorm_update_stats(ptr(nrm), ptr(nrv), ptr(rm), ptr(rv), ptr(sm), ptr(si), S, Cc, B,
                                                  float(momentum), eps, dt, current_stream(X.device)))
    return y, (nrm, nrv)


def rrule_instancenorm(x, scale, bias, act: str = "identity", epsilon: Optional[float] = None):
    """Forward + pullback Δ -> (∂x, ∂scale, ∂bias) of instancenorm with per-instance statistics (running
    statistics are not differentiated, lib/LuxLib/src/impl/normalization.jl:108)."""
    if x.dim() <= 2:
        raise AssertionError(f"`ndims(x) = {x.dim()}` must be at least > 2.")
    return rrule_groupnorm(x, scale, bias, x.shape[-2], act, epsilon)


def _gn_sizes(x, groups):
    if x.dim() < 2:
        raise DimensionMismatch("groupnorm needs at least 2 dims (channels, batch)")
    S, Cc, B = _scb(x)
    if Cc % groups != 0:
        raise ArgumentError(f"Number of channels {Cc} must be divisible by the number of groups {groups}")
    return S, Cc, B


def _groupnorm_fwd(x, scale, bias, groups, act, epsilon):
    lib = _cabi.load()
    _check_affine(scale, bias)
    X = as_colmajor(x)
    S, Cc, B = _gn_sizes(X, groups)
    if scale is not None and (scale.shape[0] != Cc or bias.shape[0] != Cc):
        raise ArgumentError("length(scale) and length(bias) must equal the number of channels")
    eps = default_epsilon(X.dtype) if epsilon is None else float(epsilon)
    dt, code, dev = dtype_code(X.dtype), act_code(act), X.device
    y = jl_empty(X.shape, X.dtype, dev)
    sm = torch.empty(groups * B, dtype=torch.float32, device=dev)
    si = torch.empty(groups * B, dtype=torch.float32, device=dev)
    sc = None if scale is None else scale.to(X.dtype)
    bi = None if bias is None else bias.to(X.dtype)
    _cabi.check(lib.lb2_groupnorm_fwd(ptr(y), ptr(sm), ptr(si), ptr(X), ptr(sc), ptr(bi), S, Cc, groups, B, eps, dt, code,
                                      current_stream(dev)))
    return y, (X, sc, bi, sm, si, S, Cc, B, dt, code)


def groupnorm(x, scale, bias, groups: int, act: str = "identity", epsilon: Optional[float] = None):
    """LuxLib.groupnorm — lib/LuxLib/src/api/groupnorm.jl:26-69."""
    return _groupnorm_fwd(x, scale, bias, groups, act, epsilon)[0]


def rrule_groupnorm(x, scale, bias, groups: int, act: str = "identity", epsilon: Optional[float] = None):
    """rrule(groupnorm_affine_normalize_internal) (lib/LuxLib/src/impl/groupnorm.jl:349-381) chained
    through mean_var. Pullback Δ -> (∂x, ∂scale, ∂bias)."""
    lib = _cabi.load()
    y, (X, sc, bi, sm, si, S, Cc, B, dt, code) = _groupnorm_fwd(x, scale, bias, groups, act, epsilon)

    def pullback(delta):
        d = as_colmajor(delta.to(X.dtype))
        dx = jl_empty(X.shape, X.dtype, X.device)
        dg = torch.empty(Cc, dtype=X.dtype, device=X.device) if sc is not None else None
        db = torch.empty(Cc, dtype=X.dtype, device=X.device) if sc is not None else None
        _, wsp, wsn = _ws(lib.lb2_groupnorm_bwd_workspace_bytes(S, Cc, groups, B), X.device)
        _cabi.check(lib.lb2_groupnorm_bwd(ptr(dx), ptr(dg), ptr(db), ptr(d), ptr(X), ptr(sc), ptr(bi), ptr(sm), ptr(si), S,
                                          Cc, groups, B, dt, code, wsp, wsn, current_stream(X.device)))
        return dx, dg, db

    return y, pullback


def _ln_rows(x, scale, bias, dims):
    """Resolves `dims` (1-based, Julia style; None, "colon", int, or a tuple) to the (D, R) row view.
    Only leading dims with scale/bias of the row shape take the fused path
    (lib/LuxLib/src/impl/layernorm.jl:16-33)."""
    _check_affine(scale, bias)
    N = x.dim()
    if dims is None:
        if scale is None:
            raise ArgumentError("`dims` must be passed explicitly if `scale` and `bias` are `nothing`")
        M = scale.dim()
        assert N > M, "`x` must have more dimensions than `scale` and `bias` when `dims` is `nothing`"
        dims = tuple(range(1, N - M + 1))
    elif dims == "colon":
        dims = tuple(range(1, N + 1))
    elif isinstance(dims, int):
        dims = (dims,)
    dims = tuple(sorted(int(d) for d in dims))
    if dims != tuple(range(1, len(dims) + 1)):
        raise ArgumentError("the fused layernorm covers leading dims only; other `dims` stay on the generic path")
    D = 1
    for d in x.shape[:len(dims)]:
        D *= d
    R = x.numel() // D if D > 0 else 0
    if scale is not None:
        lead = tuple(x.shape[:len(dims)])
        for v in (scale, bias):
            vs = tuple(v.shape)
            if vs[:len(lead)] != lead or any(d != 1 for d in vs[len(lead):]):
                raise ArgumentError("the fused layernorm needs scale / bias of the normalised shape")
    return D, R


def _layernorm_fwd(x, scale, bias, act, dims, epsilon):
    lib = _cabi.load()
    D, R = _ln_rows(x, scale, bias, dims)
    X = as_colmajor(x)
    eps = default_epsilon(X.dtype) if epsilon is None else float(epsilon)
    dt, code, dev = dtype_code(X.dtype), act_code(act), X.device
    y = jl_empty(X.shape, X.dtype, dev)
    sm = torch.empty(max(R, 1), dtype=torch.float32, device=dev)
    si = torch.empty(max(R, 1), dtype=torch.float32, device=dev)
    sc = None if scale is None else as_colmajor(scale.to(X.dtype))
    bi = None if bias is None else as_colmajor(bias.to(X.dtype))
    _cabi.check(lib.lb2_layernorm_fwd(ptr(y), ptr(sm), ptr(si), ptr(X), ptr(sc), ptr(bi), D, R, eps, dt, code,
                                      current_stream(dev)))
    return y, (X, sc, bi, sm, si, D, R, dt, code)


def layernorm(x, scale=None, bias=None, act: str = "identity", dims=None, epsilon: Optional[float] = None):
    """LuxLib.layernorm — lib/LuxLib/src/api/layernorm.jl:32-43 (op default dims = 1:N-1 is the
    caller's to pass; `dims=None` derives them from the affine rank)."""
    return _layernorm_fwd(x, scale, bias, act, dims, epsilon)[0]


def rrule_layernorm(x, scale=None, bias=None, act: str = "identity", dims=None, epsilon: Optional[float] = None):
    """Pullback Δ -> (∂x, ∂scale, ∂bias) — what broadcast AD through affine_normalize and the mean_var
    rule yields (lib/LuxLib/src/impl/normalization.jl:11-17, common_ops.jl:45-61), in one kernel."""
    lib = _cabi.load()
    y, (X, sc, bi, sm, si, D, R, dt, code) = _layernorm_fwd(x, scale, bias, act, dims, epsilon)

    def pullback(delta):
        d = as_colmajor(delta.to(X.dtype))
        dx = jl_empty(X.shape, X.dtype, X.device)
        dg = jl_empty(sc.shape, X.dtype, X.device) if sc is not None else None
        db = jl_empty(sc.shape, X.dtype, X.device) if sc is not None else None
        _, wsp, wsn = _ws(lib.lb2_layernorm_bwd_workspace_bytes(D, R), X.device)
        _cabi.check(lib.lb2_layernorm_bwd(ptr(dx), ptr(dg), ptr(db), ptr(d), ptr(X), ptr(sc), ptr(bi), ptr(sm), ptr(si), D, R,
                                          dt, code, wsp, wsn, current_stream(X.device)))
        return dx, dg, db

    return y, pullback


# --------------------------------------------------------------------------------------------
# loss
# --------------------------------------------------------------------------------------------
def rrule_mse_loss(yhat, y):
    """MSELoss()(ŷ, y) = mean(abs2.(ŷ .- y)) (src/helpers/losses.jl:659, l2_distance_loss and its derivative at
    :121-125) with its pullback: returns (loss, Δ -> ∂ŷ). Loss and gradient come from ONE pass; the loss is a
    Float32 device scalar (no synchronisation)."""
    lib = _cabi.load()
    if tuple(yhat.shape) != tuple(y.shape):
        raise DimensionMismatch("ŷ and y must have the same shape")
    yhat, y = _promote(yhat, y)
    Yh, Y = as_colmajor(yhat), as_colmajor(y)
    n = Yh.numel()
    loss = torch.empty(1, dtype=torch.float32, device=Yh.device)
    d = jl_empty(Yh.shape, Yh.dtype, Yh.device)
    _, wsp, wsn = _ws(lib.lb2_mse_loss_workspace_bytes(n), Yh.device)
    _cabi.check(lib.lb2_mse_loss(ptr(loss), ptr(d), ptr(Yh), ptr(Y), n, dtype_code(Yh.dtype), wsp, wsn, current_stream(Yh.device)))

    def pullback(delta=None):
        return d if delta is None else d * delta

    return loss, pullback


def rrule_cross_entropy_loss(yhat, y, *, logits: bool = False, label_smoothing=None, epsilon=None):
    """CrossEntropyLoss(; dims = 1, agg = mean, logits, label_smoothing, epsilon)(ŷ, y) (src/helpers/losses.jl:383-416)
    with its pullback: returns (loss, Δ -> ∂ŷ). The class dimension is the first one; all others are columns.
    `epsilon` defaults to eps(T) of the arrays' element type (src/helpers/losses.jl:104-105)."""
    lib = _cabi.load()
    if tuple(yhat.shape) != tuple(y.shape):
        raise DimensionMismatch("ŷ and y must have the same shape")
    if label_smoothing is not None and not (0 <= label_smoothing <= 1):
        raise AssertionError("0 <= label_smoothing <= 1")
    yhat, y = _promote(yhat, y)
    Yh, Y = as_colmajor(yhat), as_colmajor(y)
    K = Yh.shape[0] if Yh.dim() else 1
    B = Yh.numel() // K if K else 0
    eps = float(epsilon) if epsilon is not None else float(torch.finfo(Yh.dtype).eps)
    loss = torch.empty(1, dtype=torch.float32, device=Yh.device)
    d = jl_empty(Yh.shape, Yh.dtype, Yh.device)
    _, wsp, wsn = _ws(lib.lb2_cross_entropy_workspace_bytes(K, B), Yh.device)
    _cabi.check(lib.lb2_cross_entropy(ptr(loss), ptr(d), ptr(Yh), ptr(Y), K, B, 1 if logits else 0, float(label_smoothing or 0.0), eps,
                                      dtype_code(Yh.dtype), wsp, wsn, current_stream(Yh.device)))

    def pullback(delta=None):
        return d if delta is None else d * delta

    return loss, pullback


def cross_entropy_loss(yhat, y, **kw):
    """CrossEntropyLoss(...)(ŷ, y) as a Float32 device scalar."""
    return rrule_cross_entropy_loss(yhat, y, **kw)[0]


def mse_loss(yhat, y):
    """MSELoss()(ŷ, y) as a Float32 device scalar."""
    return rrule_mse_loss(yhat, y)[0]
