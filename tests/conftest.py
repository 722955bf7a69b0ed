"""Shared pytest configuration: the `gpu` marker and import paths."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "lux.jl_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        have_gpu = torch.cuda.is_available()
    except Exception:
        have_gpu = False
    if have_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def pytest_terminal_summary(terminalreporter, exitstatus, config):
    """Write the measured parity errors and print the worst one per (test, tensor, dtype)."""
    import parity_report
    path = parity_report.write()
    if path is None:
        return
    tr = terminalreporter
    tr.write_sep("-", f"parity errors measured ({len(parity_report.RECORDS)} comparisons, written to {path})")
    for (fn, tensor, dt), r in sorted(parity_report.worst_by_function().items()):
        tr.write_line(f"{fn:62s} {tensor:28s} {dt:5s} rel-L2 {r['rel_l2']:.3e}  (tol {r['tol']:.0e})")
