import json
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden_dir():
    return os.path.join(ROOT, "tests", "golden")


def pytest_terminal_summary(terminalreporter):
    """Measured parity of every f16 comparison of the session: the end-to-end ones (those that allow a fraction of elements
    outside the per-element rule) line by line, the zero-tolerance ones as a count with their worst case."""
    import tolerance
    recs = tolerance.RECORDS
    if not recs:
        return
    tr = terminalreporter
    tr.section("parity measurements (f16 rule: rel 2e-2 OR abs 2e-3 per element)")
    e2e = [r for r in recs if r["allowed_fail_fraction"] > 0]
    strict = [r for r in recs if r["allowed_fail_fraction"] == 0]
    for r in e2e:
        tr.write_line(f"{r['what'][:70]:70s} outside {r['fail_fraction']:.2e} (allowed {r['allowed_fail_fraction']:.0e})  "
                      f"max|err| {r['max_abs_err']:.2e}  rel-L2 {r['rel_l2']:.2e}  n={r['elements']}")
    if strict:
        worst = max(strict, key=lambda r: r["rel_l2"])
        tr.write_line(f"{len(strict)} comparisons with ZERO elements allowed outside: all passed; worst rel-L2 {worst['rel_l2']:.2e} "
                      f"({worst['what'][:60]}), largest abs err {max(r['max_abs_err'] for r in strict):.2e}")
    path = os.environ.get("B200_PARITY_REPORT")
    if path:
        with open(path, "w") as f:
            json.dump(recs, f, indent=1)
