"""Error metrics shared by the parity tests."""
import numpy as np

FP32_TOL = 1e-5      # max |a-b| / max |b|, the fp32 bar of the training-step path
FP16_TOL = 1e-2      # same metric for fp16 storage with fp32 accumulation
# Element-wise bar: |a-b| <= ELEMENTWISE_FACTOR * tol * max(|b|, 1e-2 max|b|).  With factor 1 the bar is 100 times tighter than
# the max-norm bar on small elements and flags plain fp32 reordering noise: two fp32 evaluations of the same sums in different
# orders (this repository's CPU restatement against the reference's PyTorch golden model of attention; a warp-tree GEMV
# against the reference's sequential loop) measure 2e-5 .. 3e-5 by it, 3xTF32 products and chains of GEMMs with cancellation
# (attention backward, the 8-layer network's gradients) up to 1.5e-4 at tol 1e-5.  Factor 30 keeps the point of the bar:
# on elements below a hundredth of the largest the absolute error allowed is 0.3 * tol * max|b|, three times less than the
# max-norm bar allows, and a region of small values that is simply wrong is off by order one.
ELEMENTWISE_FACTOR = 30.0


def rel_err(a, b):
    a = np.asarray(a, np.float64).ravel(); b = np.asarray(b, np.float64).ravel()
    assert a.shape == b.shape, (a.shape, b.shape)
    den = np.abs(b).max()
    if den == 0:
        return float(np.abs(a).max())
    return float(np.abs(a - b).max() / den)


def elementwise_err(a, b):
    """max over elements of |a-b| / max(|b|, 1e-2 max|b|): a relative error per element whose denominator
    never drops below one hundredth of the tensor's largest magnitude (pure element-wise relative error is
    meaningless next to zero); catches a wrong region of small values that the max-norm metric lets through"""
    a = np.asarray(a, np.float64).ravel(); b = np.asarray(b, np.float64).ravel()
    assert a.shape == b.shape, (a.shape, b.shape)
    top = np.abs(b).max() if b.size else 0.0
    if top == 0:
        return float(np.abs(a).max()) if a.size else 0.0
    return float((np.abs(a - b) / np.maximum(np.abs(b), 1e-2 * top)).max())


def assert_close(a, b, tol, what="", elem_tol=None):
    """both bars of the training-step path: max|a-b| / max|b| <= tol for the tensor, and
    |a-b| <= tol * max(|b|, 1e-2 max|b|) for every element"""
    assert np.all(np.isfinite(np.asarray(a, np.float64))), "%s: non-finite values" % what
    e = rel_err(a, b)
    assert e <= tol, "%s: rel err %.3e > %.1e" % (what, e, tol)
    ee = elementwise_err(a, b)
    et = ELEMENTWISE_FACTOR * tol if elem_tol is None else elem_tol       # a looser element-wise bar is stated, with the measured value, at the call
    assert ee <= et, "%s: element-wise err %.3e > %.1e (denominator max(|b|, 1e-2 max|b|))" % (what, ee, et)
    return e


def assert_exact(a, b, what=""):
    a = np.asarray(a); b = np.asarray(b)
    assert a.shape == b.shape and a.dtype == b.dtype, (what, a.shape, b.shape, a.dtype, b.dtype)
    assert a.tobytes() == b.tobytes(), "%s: not bit-exact (%d elements differ)" % (what, int((a != b).sum()))


def seeded(seed):
    return np.random.default_rng(seed)
