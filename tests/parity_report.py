"""Record of the errors the GPU parity tests actually measured.

Every comparison of a device result with the CPU oracle calls `record(...)`; at the end of the pytest
session `tests/conftest.py` writes all records as JSON lines (one per comparison:
`{"test", "tensor", "dtype", "rel_l2", "tol", ...}`) to the file named by the environment variable
`LB2_PARITY_REPORT` (default: `parity_report.jsonl` in the current directory) and prints the worst figure
per (test function, tensor, dtype), so that the distance from the tolerance is on record and not only the
fact that an assertion held.
"""
import json
import os

RECORDS = []


def current_test():
    name = os.environ.get("PYTEST_CURRENT_TEST", "?")
    return name.rsplit(" ", 1)[0]


def record(tensor, dtype, rel_l2, tol, **extra):
    rec = {"test": current_test(), "tensor": tensor, "dtype": dtype, "rel_l2": float(rel_l2), "tol": float(tol)}
    rec.update(extra)
    RECORDS.append(rec)
    return rec


def worst_by_function():
    """{(test function without parameters, tensor, dtype): record with the largest rel_l2 / tol}"""
    worst = {}
    for r in RECORDS:
        fn = r["test"].split("::")[-1].split("[")[0]
        key = (fn, r["tensor"], r["dtype"])
        if key not in worst or r["rel_l2"] / r["tol"] > worst[key]["rel_l2"] / worst[key]["tol"]:
            worst[key] = r
    return worst


def write(path=None):
    path = path or os.environ.get("LB2_PARITY_REPORT", "parity_report.jsonl")
    if not RECORDS:
        return None
    with open(path, "w") as f:
        for r in RECORDS:
            f.write(json.dumps(r) + "\n")
    return path
