"""Comparison metric shared by the parity tests.

Per tensor, against the reference (b):  max|a-b| / max|b| <= tol  and  ||a-b||2 / ||b||2 <= tol.
The tolerance for tensor-core results is 1e-3 (tf32 operands, fp32 accumulation).
"""

import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
TOL = 1e-3


def golden(name):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


def errors(a, b, floor=0.0):
    """`floor`: a lower bound for both denominators, as (max-abs, rms) of a larger tensor this
    one is a part of -- e.g. the key-bias gradient of an attention layer is exactly zero in
    exact arithmetic, so it can only be judged against the scale of the whole gradient."""
    a = np.asarray(a, dtype=np.float64).ravel()
    b = np.asarray(b, dtype=np.float64).ravel()
    assert a.shape == b.shape, (a.shape, b.shape)
    max_err = np.abs(a - b).max() / max(np.abs(b).max(), floor, 1e-30)
    l2_err = np.linalg.norm(a - b) / max(np.linalg.norm(b), floor * np.sqrt(a.size), 1e-30)
    return float(max_err), float(l2_err)


def assert_close(a, b, tol=TOL, what="", floor=0.0):
    assert np.all(np.isfinite(np.asarray(a, dtype=np.float64))), f"{what}: non-finite values"
    max_err, l2_err = errors(a, b, floor)
    assert max_err <= tol and l2_err <= tol, f"{what}: max-rel {max_err:.3e}, l2-rel {l2_err:.3e} > {tol:.1e}"
    return max_err, l2_err
