"""Comparison rules shared by the parity tests.

* ``assert_close_f16``: the rule stated for this path — an element passes when EITHER
  |a-e| <= 2e-3 OR |a-e| <= 2e-2 * |e| (f16 activations, fp32 state).
* ``rel_l2``: the reference's global relative-L2 metric for f16 results
  (tests/test_tools.hpp:77-103): sqrt(sum((a-e)^2) / sum(e^2 + 1e-8)).
* ``assert_abs``: the reference's default absolute rule for fp32 ops (tests/test_tools.hpp:24-43), 1e-3.
"""
import numpy as np

REL = 2e-2
ABS = 2e-3


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
    return float(bad.mean()), float(err.max() if err.size else 0.0)


def assert_close_f16(a, e, what="", rel=REL, abs_=ABS, max_fail_fraction=0.0):
    assert a.shape == e.shape, (what, a.shape, e.shape)
    frac, mx = fail_fraction(a, e, rel, abs_)
    assert frac <= max_fail_fraction, f"{what}: {frac:.3e} of elements outside rel {rel} / abs {abs_} (max abs err {mx:.3e}, rel-L2 {rel_l2(a, e):.3e})"


def assert_abs(a, e, what="", tol=1e-3):
    assert a.shape == e.shape, (what, a.shape, e.shape)
    err = np.abs(np.asarray(a, np.float64) - np.asarray(e, np.float64))
    assert np.isfinite(np.asarray(a)).all() and err.max() < tol, f"{what}: max abs err {err.max():.3e} >= {tol}"
