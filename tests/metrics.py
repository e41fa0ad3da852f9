"""Error metrics shared by the parity tests."""
import numpy as np

FP32_TOL = 1e-5      # max |a-b| / max |b|, the fp32 bar of the training-step path
FP16_TOL = 1e-2      # same metric for fp16 storage with fp32 accumulation


def rel_err(a, b):
    a = np.asarray(a, np.float64).ravel(); b = np.asarray(b, np.float64).ravel()
    assert a.shape == b.shape, (a.shape, b.shape)
    den = np.abs(b).max()
    if den == 0:
        return float(np.abs(a).max())
    return float(np.abs(a - b).max() / den)


def assert_close(a, b, tol, what=""):
    assert np.all(np.isfinite(np.asarray(a, np.float64))), "%s: non-finite values" % what
    e = rel_err(a, b)
    assert e <= tol, "%s: rel err %.3e > %.1e" % (what, e, tol)
    return e


def assert_exact(a, b, what=""):
    a = np.asarray(a); b = np.asarray(b)
    assert a.shape == b.shape and a.dtype == b.dtype, (what, a.shape, b.shape, a.dtype, b.dtype)
    assert a.tobytes() == b.tobytes(), "%s: not bit-exact (%d elements differ)" % (what, int((a != b).sum()))


def seeded(seed):
    return np.random.default_rng(seed)
