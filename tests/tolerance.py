"""Comparison rules shared by the parity tests.

* ``assert_close_f16``: the rule stated for this path — an element passes when EITHER
  |a-e| <= 2e-3 OR |a-e| <= 2e-2 * |e| (f16 activations, fp32 state). Per-operator checks allow ZERO elements outside.
  End-to-end checks (several f16 roundings between the input and the compared tensor) may allow a small fraction outside
  (``max_fail_fraction``); for those, two further bounds always apply: NO element may lie outside ``outer`` times the rule
  (so the failing elements are near misses, not arbitrary values), and the global relative-L2 error must stay below
  ``max_rel_l2``.
* ``rel_l2``: the reference's global relative-L2 metric for f16 results
  (tests/test_tools.hpp:77-103): sqrt(sum((a-e)^2) / sum(e^2 + 1e-8)); the reference accepts 1e-2.
* ``assert_abs``: the reference's default absolute rule for fp32 ops (tests/test_tools.hpp:24-43), 1e-3.

Every ``assert_close_f16`` call is recorded (measured fraction outside, largest error, rel-L2 beside what was allowed); the
session prints the records of the end-to-end checks at its end and writes all of them to the file named by the environment
variable B200_PARITY_REPORT, so that the slack of every tolerance is visible.
"""
import os

import numpy as np

REL = 2e-2
ABS = 2e-3
OUTER = 5.0
MAX_REL_L2 = 2e-3

RECORDS = []


def rel_l2(a, e):
    a = np.asarray(a, np.float64)
    e = np.asarray(e, np.float64)
    return float(np.sqrt(((a - e) ** 2).sum() / (e ** 2 + 1e-8).sum()))


def fail_fraction(a, e, rel=REL, abs_=ABS):
    a = np.asarray(a, np.float64)
    e = np.asarray(e, np.float64)
    err = np.abs(a - e)
    bad = (err > abs_) & (err > rel * np.abs(e))
    bad |= ~np.isfinite(a)
    return float(bad.mean()) if bad.size else 0.0, float(err.max() if err.size else 0.0)


def assert_close_f16(a, e, what="", rel=REL, abs_=ABS, max_fail_fraction=0.0, outer=OUTER, max_rel_l2=MAX_REL_L2):
    assert a.shape == e.shape, (what, a.shape, e.shape)
    frac, mx = fail_fraction(a, e, rel, abs_)
    l2 = rel_l2(a, e)
    outer_frac = fail_fraction(a, e, rel * outer, abs_ * outer)[0] if max_fail_fraction > 0 else frac
    RECORDS.append({"test": os.environ.get("PYTEST_CURRENT_TEST", "").split(" ")[0], "what": what, "elements": int(np.asarray(a).size),
                    "fail_fraction": frac, "allowed_fail_fraction": max_fail_fraction, "max_abs_err": mx, "rel_l2": l2,
                    "rel": rel, "abs": abs_, "fraction_outside_outer_bound": outer_frac})
    msg = f"{what}: {frac:.3e} of elements outside rel {rel} / abs {abs_} (max abs err {mx:.3e}, rel-L2 {l2:.3e})"
    assert frac <= max_fail_fraction, msg
    if max_fail_fraction > 0:
        assert outer_frac == 0.0, f"{what}: {outer_frac:.3e} of elements outside {outer} x the rule; " + msg
        assert l2 < max_rel_l2, f"{what}: rel-L2 {l2:.3e} >= {max_rel_l2}; " + msg


def assert_abs(a, e, what="", tol=1e-3):
    assert a.shape == e.shape, (what, a.shape, e.shape)
    err = np.abs(np.asarray(a, np.float64) - np.asarray(e, np.float64))
    assert np.isfinite(np.asarray(a)).all() and err.max() < tol, f"{what}: max abs err {err.max():.3e} >= {tol}"
