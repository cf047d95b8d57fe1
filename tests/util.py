"""Shared helpers of the parity tests."""
import numpy as np

ABS_TOL = 2e-3   # attention outputs: |gpu - ref| <= ABS_TOL + REL_TOL * |ref|  (fp32 accumulate)
REL_TOL = 1e-3


def assert_close(got, want, what=""):
    got = np.asarray(got, dtype=np.float32).reshape(-1)
    want = np.asarray(want, dtype=np.float32).reshape(-1)
    assert got.shape == want.shape, (got.shape, want.shape)
    assert np.all(np.isfinite(got)), f"{what}: non-finite output"
    err = np.abs(got - want)
    bound = ABS_TOL + REL_TOL * np.abs(want)
    bad = err > bound
    assert not bad.any(), (f"{what}: {bad.sum()} of {bad.size} outside tolerance; max abs err {err.max():.3e} "
                           f"at {err.argmax()} (got {got[err.argmax()]}, want {want[err.argmax()]})")
    return float(err.max())


def assert_bits_equal(got, want, what=""):
    got = np.ascontiguousarray(got)
    want = np.ascontiguousarray(want)
    assert got.nbytes == want.nbytes, (what, got.nbytes, want.nbytes)
    a = got.view(np.uint8).reshape(-1)
    b = want.view(np.uint8).reshape(-1)
    diff = np.nonzero(a != b)[0]
    assert diff.size == 0, f"{what}: {diff.size} bytes differ, first at byte {diff[0]} ({a[diff[0]]} vs {b[diff[0]]})"


def normal(seed, shape, scale=1.0):
    return (np.random.default_rng(seed).standard_normal(shape, dtype=np.float32) * np.float32(scale)).astype(np.float32)
