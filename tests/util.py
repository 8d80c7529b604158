"""Shared helpers of the test-suite: layouts, tolerances, oracle access."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from oracle import oracle_c, oracle_np  # noqa: E402

# acceptance tolerances of the path in complex64 (relative to max|ref| and to ||ref||_2)
MAX_REL_TOL = 1e-4
REL_L2_TOL = 1e-5


def to_reference_layout(x_logical):
    """logical x[B, K, ...] -> reference memory order [K, B, ...] (channel outermost)."""
    return np.ascontiguousarray(np.swapaxes(x_logical, 0, 1))


def from_reference_layout(y_ref_layout):
    """[N, B, ...] -> logical [B, N, ...]."""
    return np.swapaxes(y_ref_layout, 0, 1)


def w_reference_layout(w_logical):
    """logical w[K, N] -> reference order: element (k, n) at k + n*K, i.e. an [N, K] array."""
    return np.ascontiguousarray(w_logical.T)


def assert_close(test, ref, what="", max_rel=MAX_REL_TOL, rel_l2=REL_L2_TOL):
    mr, l2 = oracle_np.errors(test, ref)
    assert mr <= max_rel and l2 <= rel_l2, "%s: max_rel=%.3e (tol %.1e) rel_l2=%.3e (tol %.1e)" % (what, mr, max_rel, l2, rel_l2)
    return mr, l2
