"""The allocation-free BatchNorm entry point (scratch built into the library) must give what the
workspace-taking entry point gives. Collected last on purpose (file name), so a run that stops at
the first failure has already exercised everything else. Called straight through the C ABI."""
import numpy as np
import pytest
import torch

import luxlib_b200 as L
from luxlib_b200 import _cabi

pytestmark = pytest.mark.gpu


def _run(lib, static: bool, x, gamma, beta, rmean, rvar, S, C, B, act, dtype=None):
    dev = x.device
    dtype = _cabi.F32 if dtype is None else dtype
    y = torch.empty_like(x)
    sm = torch.empty(C, dtype=torch.float32, device=dev)
    si = torch.empty(C, dtype=torch.float32, device=dev)
    have_stats = rmean is not None
    nrm = torch.empty_like(rmean) if have_stats else None
    nrv = torch.empty_like(rvar) if have_stats else None
    p = lambda t: None if t is None else t.data_ptr()
    stream = torch.cuda.current_stream(dev).cuda_stream
    common = (y.data_ptr(), sm.data_ptr(), si.data_ptr(), p(nrm), p(nrv), x.data_ptr(), gamma.data_ptr(),
              beta.data_ptr(), p(rmean), p(rvar), S, C, B, 0.1, 1e-5, dtype, act)
    if static:
        rc = lib.lb2_batchnorm_fwd_train_static(*common, stream)
    else:
        n = lib.lb2_batchnorm_workspace_bytes(S, C, B)
        ws = torch.empty(n, dtype=torch.uint8, device=dev)
        rc = lib.lb2_batchnorm_fwd_train(*common, ws.data_ptr(), n, stream)
    assert rc == _cabi.OK, lib.lb2_last_error_string()
    torch.cuda.synchronize()
    outs = [y, sm, si] + ([nrm, nrv] if have_stats else [])
    return [t.clone() for t in outs]


NAMES = ("y", "save_mean", "save_invstd", "running_mean", "running_var")
# (seed, (S, C, B), activation, storage type, running statistics given): two small Float32 problems (three-kernel
# path), a Float32 tensor above 16 MiB (single cooperative launch; its barrier counters and per-CTA partials live in
# the built-in scratch too), a bf16 problem and one without running statistics
CASES = (
    (0, (196, 64, 32), _cabi.ACT_RELU, "f32", True),
    (1, (49, 48, 16), _cabi.ACT_IDENTITY, "f32", True),
    (2, (96 * 96, 40, 24), _cabi.ACT_RELU, "f32", True),
    (3, (256, 32, 24), _cabi.ACT_RELU, "bf16", True),
    (4, (100, 24, 8), _cabi.ACT_IDENTITY, "f32", False),
)


def test_static_scratch_batchnorm_matches_the_workspace_entry_point_twice_in_a_row():
    lib = _cabi.load()
    # different problems back to back, each run twice: every call finds the previous call's leftovers in the scratch
    for seed, (S, C, B), act, dt, stats in CASES:
        tdt = torch.float32 if dt == "f32" else torch.bfloat16
        g = torch.Generator(device="cuda").manual_seed(seed)
        x = (torch.randn(B, C, S, device="cuda", generator=g) * 1.7 + 0.4).to(tdt)   # memory order of a column-major (S, C, B)
        gamma = (torch.rand(C, device="cuda", generator=g) + 0.5).to(tdt)
        beta = (torch.randn(C, device="cuda", generator=g) * 0.1).to(tdt)
        rmean = torch.zeros(C, device="cuda", dtype=tdt) if stats else None
        rvar = torch.ones(C, device="cuda", dtype=tdt) if stats else None
        code = _cabi.F32 if dt == "f32" else _cabi.BF16
        assert lib.lb2_batchnorm_workspace_bytes(S, C, B) <= (4 << 20)
        want = _run(lib, False, x, gamma, beta, rmean, rvar, S, C, B, act, code)
        for _ in range(2):
            got = _run(lib, True, x, gamma, beta, rmean, rvar, S, C, B, act, code)
            for w, gt, name in zip(want, got, NAMES):
                err = (gt.double() - w.double()).norm() / w.double().norm()
                # same tolerances as the parity tests: 1e-5 for Float32 storage, 1e-2 for bf16 storage
                assert err <= (1e-5 if dt == "f32" or name.startswith("save") else 1e-2), f"{dt} {S}x{C}x{B} {name}: rel-L2 {err:.3e}"
    assert lib.lb2_poll_device_status(None) == 0


def test_static_scratch_settles_argument_errors_and_empty_problems_first():
    lib = _cabi.load()
    # a null tensor is an argument error and an empty problem is OK; neither needs the scratch
    assert lib.lb2_batchnorm_fwd_train_static(None, None, None, None, None, None, None, None, None, None, 4, 4, 4, 0.1, 1e-5,
                                              _cabi.F32, _cabi.ACT_IDENTITY, None) == _cabi.BAD_ARG
    assert lib.lb2_batchnorm_fwd_train_static(None, None, None, None, None, None, None, None, None, None, 0, 4, 4, 0.1, 1e-5,
                                              _cabi.F32, _cabi.ACT_IDENTITY, None) == _cabi.OK


def test_static_scratch_rejects_problems_beyond_its_size():
    lib = _cabi.load()
    S, C, B = 1, 1 << 18, 2   # needs more scratch than the built-in 4 MiB
    assert lib.lb2_batchnorm_workspace_bytes(S, C, B) > (4 << 20)
    rc = lib.lb2_batchnorm_fwd_train_static(16, 16, 16, None, None, 16, None, None, None, None, S, C, B, 0.1, 1e-5,
                                            _cabi.F32, _cabi.ACT_IDENTITY, None)
    assert rc == _cabi.WORKSPACE_TOO_SMALL
    assert b"built-in scratch" in lib.lb2_last_error_string()
