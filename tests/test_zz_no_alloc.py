"""The allocation-free BatchNorm entry point (scratch built into the library) must give what the
workspace-taking entry point gives. Collected last on purpose (file name), so a run that stops at
the first failure has already exercised everything else. Called straight through the C ABI."""
import numpy as np
import pytest
import torch

import luxlib_b200 as L
from luxlib_b200 import _cabi

pytestmark = pytest.mark.gpu


def _run(lib, static: bool, x, gamma, beta, rmean, rvar, S, C, B, act):
    dev = x.device
    y = torch.empty_like(x)
    sm = torch.empty(C, dtype=torch.float32, device=dev)
    si = torch.empty(C, dtype=torch.float32, device=dev)
    nrm, nrv = torch.empty_like(rmean), torch.empty_like(rvar)
    stream = torch.cuda.current_stream(dev).cuda_stream
    common = (y.data_ptr(), sm.data_ptr(), si.data_ptr(), nrm.data_ptr(), nrv.data_ptr(), x.data_ptr(), gamma.data_ptr(),
              beta.data_ptr(), rmean.data_ptr(), rvar.data_ptr(), S, C, B, 0.1, 1e-5, _cabi.F32, act)
    if static:
        rc = lib.lb2_batchnorm_fwd_train_static(*common, stream)
    else:
        n = lib.lb2_batchnorm_workspace_bytes(S, C, B)
        ws = torch.empty(n, dtype=torch.uint8, device=dev)
        rc = lib.lb2_batchnorm_fwd_train(*common, ws.data_ptr(), n, stream)
    assert rc == _cabi.OK, lib.lb2_last_error_string()
    torch.cuda.synchronize()
    return [t.clone() for t in (y, sm, si, nrm, nrv)]


def test_static_scratch_batchnorm_matches_the_workspace_entry_point_twice_in_a_row():
    lib = _cabi.load()
    # two different problems back to back: the second call finds the first call's leftovers in the scratch
    for seed, (S, C, B), act in ((0, (196, 64, 32), _cabi.ACT_RELU), (1, (49, 48, 16), _cabi.ACT_IDENTITY)):
        g = torch.Generator(device="cuda").manual_seed(seed)
        x = torch.randn(B, C, S, device="cuda", generator=g) * 1.7 + 0.4      # memory order of a column-major (S, C, B)
        gamma = torch.rand(C, device="cuda", generator=g) + 0.5
        beta = torch.randn(C, device="cuda", generator=g) * 0.1
        rmean, rvar = torch.zeros(C, device="cuda"), torch.ones(C, device="cuda")
        want = _run(lib, False, x, gamma, beta, rmean, rvar, S, C, B, act)
        for _ in range(2):
            got = _run(lib, True, x, gamma, beta, rmean, rvar, S, C, B, act)
            for w, gt, name in zip(want, got, ("y", "save_mean", "save_invstd", "running_mean", "running_var")):
                err = (gt.double() - w.double()).norm() / w.double().norm()
                assert err <= 1e-5, f"{name}: rel-L2 {err:.3e}"   # same tolerance as the fp32 parity tests


def test_static_scratch_rejects_problems_beyond_its_size():
    lib = _cabi.load()
    S, C, B = 1, 1 << 18, 2   # needs more scratch than the built-in 4 MiB
    assert lib.lb2_batchnorm_workspace_bytes(S, C, B) > (4 << 20)
    rc = lib.lb2_batchnorm_fwd_train_static(16, 16, 16, None, None, 16, None, None, None, None, S, C, B, 0.1, 1e-5,
                                            _cabi.F32, _cabi.ACT_IDENTITY, None)
    assert rc == _cabi.WORKSPACE_TOO_SMALL
    assert b"built-in scratch" in lib.lb2_last_error_string()
