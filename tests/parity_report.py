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


def summarize(path):
    """Markdown summary of a report file: per (test function, dtype) the number of comparisons and the worst one."""
    global RECORDS
    with open(path) as f:
        RECORDS = [json.loads(line) for line in f if line.strip()]
    groups = {}
    for r in RECORDS:
        fn = r["test"].split("::")[-1].split("[")[0]
        groups.setdefault((fn, r["dtype"]), []).append(r)
    rows = ["| test | dtype | comparisons | worst rel-L2 | tolerance | worst tensor | note |", "|---|---|---|---|---|---|---|"]
    for (fn, dt), rs in sorted(groups.items()):
        r = max(rs, key=lambda q: q["rel_l2"] / q["tol"])
        note = r.get("judged", "")
        if "rel_l2_plain" in r:
            note += f" (plain {r['rel_l2_plain']:.2e}, cancellation {r.get('cancellation', float('nan')):.3g})"
        rows.append(f"| {fn} | {dt} | {len(rs)} | {r['rel_l2']:.2e} | {r['tol']:.0e} | {r['tensor']} | {note} |")
    head = f"{len(RECORDS)} comparisons; worst over all Float32 comparisons relative to their tolerance: "
    f32 = [r for r in RECORDS if r["dtype"] == "f32"]
    bf = [r for r in RECORDS if r["dtype"] == "bf16"]
    w32 = max(f32, key=lambda r: r["rel_l2"] / r["tol"]) if f32 else None
    wbf = max(bf, key=lambda r: r["rel_l2"] / r["tol"]) if bf else None
    if w32:
        head += f"{w32['rel_l2']:.2e} of {w32['tol']:.0e} ({w32['test'].split('::')[-1]}, {w32['tensor']})"
    if wbf:
        head += f"; bf16: {wbf['rel_l2']:.2e} of {wbf['tol']:.0e} ({wbf['test'].split('::')[-1]}, {wbf['tensor']})"
    return head + "\n\n" + "\n".join(rows) + "\n"


if __name__ == "__main__":
    import sys
    print(summarize(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("LB2_PARITY_REPORT", "parity_report.jsonl")))
