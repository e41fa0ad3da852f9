"""GPU: the allocation-free Linear input gradient (trainlib_linear_fp32_bw_input_grads_noalloc).

It exists for hosts that cannot let this library allocate device memory (the application's own pool owns
the device, or the memory budget is fixed at start-up): its scratch is a fixed array inside the library.
The test calls it through the C ABI twice in a row, on different inputs, and compares each result with the
ordinary entry point pulp_linear_fp32_bw_input_grads_cl (which takes its scratch from the staging arena) and with
the CPU oracle (both GPU entry points share their kernels, so only the oracle can catch a fault in those);
the second call must not be disturbed by what the first one left in the array.  Collected last on purpose."""
import numpy as np
import pytest

from abi_runner import AbiRunner
from metrics import FP32_TOL, assert_close, seeded

pytestmark = pytest.mark.gpu
F = np.float32


def reference_dx(pkg, lib, W, dy):
    r = AbiRunner(pkg, lib, device=True)
    out, inn = W.shape
    res = r.linear(W, np.zeros(inn, F), dy)
    r.close()
    return res["dx"]


@pytest.mark.parametrize("shapes", [[(1024, 4096), (333, 77)], [(64, 256), (4096, 1024)]])
def test_two_calls_in_a_row_match_the_allocating_entry_point(pkg, gpulib, oracle, shapes):
    rng = seeded(123)
    for out, inn in shapes:
        W = (rng.standard_normal((out, inn)) / np.sqrt(inn)).astype(F); dy = rng.standard_normal(out).astype(F)
        want = reference_dx(pkg, gpulib, W, dy)
        assert_close(want, oracle.linear(W, np.zeros(inn, F), dy)["dx"].reshape(want.shape), FP32_TOL, "allocating entry point vs CPU oracle, %dx%d" % (out, inn))
        dW, ddy, ddx = pkg.DeviceBuffer(gpulib, W), pkg.DeviceBuffer(gpulib, dy), pkg.DeviceBuffer(gpulib, nbytes=4 * inn)
        rc = gpulib.trainlib_linear_fp32_bw_input_grads_noalloc(dW.ptr, ddy.ptr, ddx.ptr, out, inn, gpulib.trainlib_stream())
        assert rc == 0, gpulib.trainlib_last_error_string().decode()
        gpulib.trainlib_synchronize()
        got = ddx.download(F, (inn,))
        assert_close(got, want, FP32_TOL, "no-alloc dx for %dx%d" % (out, inn))
        for b in (dW, ddy, ddx):
            b.free()


def test_the_widest_accepted_layer(pkg, gpulib, oracle):
    """in = 1 048 576, the largest width the fixed array serves (one slab of partial sums fills it exactly), against the CPU oracle"""
    rng = seeded(124)
    out, inn = 8, 1 << 20
    W = (rng.standard_normal((out, inn)) / 32).astype(F); dy = rng.standard_normal(out).astype(F)
    dW, ddy, ddx = pkg.DeviceBuffer(gpulib, W), pkg.DeviceBuffer(gpulib, dy), pkg.DeviceBuffer(gpulib, nbytes=4 * inn)
    rc = gpulib.trainlib_linear_fp32_bw_input_grads_noalloc(dW.ptr, ddy.ptr, ddx.ptr, out, inn, gpulib.trainlib_stream())
    assert rc == 0, gpulib.trainlib_last_error_string().decode()
    gpulib.trainlib_synchronize()
    assert_close(ddx.download(F, (inn,)), oracle.linear(W, np.zeros(inn, F), dy)["dx"].ravel(), FP32_TOL, "no-alloc dx at the capacity limit")
    for b in (dW, ddy, ddx):
        b.free()


def test_sizes_beyond_the_fixed_scratch_are_refused(pkg, gpulib):
    d = pkg.DeviceBuffer(gpulib, nbytes=64)
    rc = gpulib.trainlib_linear_fp32_bw_input_grads_noalloc(d.ptr, d.ptr, d.ptr, 4, (1 << 20) + 1, None)
    assert rc == 5                                   # TL_ERR_TOO_LARGE, nothing launched
    assert "exceeds the fixed scratch" in gpulib.trainlib_last_error_string().decode()
    gpulib.trainlib_clear_error()
    d.free()
