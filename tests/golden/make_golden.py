"""Regenerates tests/golden/fixed_array_cases.npz.

Inputs are the reference test-suite's deterministic arrays (`generate_fixed_array`,
lib/LuxLib/test/shared_testsetup.jl:69-73: reshape((1:n)/n, size) in column-major order) on the
shapes its conv / batchnorm / layernorm / groupnorm tests use
(lib/LuxLib/test/common_ops/conv_tests.jl:87-117, normalization/batchnorm_tests.jl:128-141,
normalization/layernorm_tests.jl:80-98). Expected outputs come from the CPU oracle in float64 and
are stored as float32. The reference itself cannot run here (no Julia), so these vectors pin the
oracle + CUDA path against drift, not against LuxLib binaries.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import luxlib_oracle as O  # noqa: E402

CONV = [  # kernel, padding, stride, groups  (conv_tests.jl:87-92), x = 4x4x4x2 -> 8 channels
    ((3, 3), 0, 1, 1), ((3, 3), 0, 1, 2), ((3, 3), 2, 1, 1), ((3, 3), 0, 2, 1),
]


def cases():
    out = {}
    f = lambda shp: O.generate_fixed_array(shp, np.float64)
    for i, (k, pad, stride, groups) in enumerate(CONV):
        x, w, b = f((4, 4, 4, 2)), f(k + (4 // groups, 8)), f((8,))
        cd = O.ConvDims.make(2, stride, pad, 1, groups, False)
        for act in ("identity", "sigmoid", "gelu"):
            y, pb = O.fused_conv_rrule(act, w, x, b, cd)
            dw, dx, db = pb(np.ones_like(y) * 0.5 + y * 0.25)
            out[f"conv{i}_{act}"] = dict(y=y, dw=dw, dx=dx, db=db)
    for shp in ((4, 4, 6, 2), (8, 2)):
        c = shp[-2]
        x, g, b = f(shp), f((c,)), f((c,))
        rm, rv = np.zeros(c), np.ones(c)
        for act in ("identity", "sigmoid"):
            z, (nrm, nrv), pb = O.batchnorm_rrule(x, g, b, rm, rv, True, act, 0.9, 1e-5)
            dx, dg, dbt = pb(np.ones_like(z) * 0.5 + z * 0.25)
            out[f"bn{'x'.join(map(str, shp))}_{act}"] = dict(y=z, rmean=nrm, rvar=nrv, dx=dx, dgamma=dg, dbeta=dbt)
    for shp, nd in (((4, 4, 6, 2), 3), ((6, 3), 1)):
        x = f(shp)
        ashape = shp[:nd] + (1,) * (len(shp) - nd)
        g, b = f(ashape), f(ashape)
        z, pb = O.layernorm_rrule(x, g, b, "identity", tuple(range(nd)), 1e-5)
        dx, dg, dbt = pb(np.ones_like(z) * 0.5 + z * 0.25)
        out[f"ln{'x'.join(map(str, shp))}"] = dict(y=z, dx=dx, dgamma=dg, dbeta=dbt)
    for shp, groups in (((4, 4, 6, 2), 3), ((6, 2), 2)):
        x, g, b = f(shp), f((6,)), f((6,))
        z, pb = O.groupnorm_rrule(x, g, b, groups, "identity", 1e-5)
        dx, dg, dbt = pb(np.ones_like(z) * 0.5 + z * 0.25)
        out[f"gn{'x'.join(map(str, shp))}_g{groups}"] = dict(y=z, dx=dx, dgamma=dg, dbeta=dbt)
    return out


if __name__ == "__main__":
    flat = {}
    for name, d in cases().items():
        for k, v in d.items():
            flat[f"{name}/{k}"] = np.asarray(v, dtype=np.float32)
    np.savez_compressed(os.path.join(HERE, "fixed_array_cases.npz"), **flat)
    print(len(flat), "arrays written")
