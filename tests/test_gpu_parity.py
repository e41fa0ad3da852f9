"""GPU parity: libtrainlib_b200 called through the C ABI, against (1) the committed golden vectors
of the reference's own C code, (2) the CPU oracle on seeded inputs at further sizes, and (3) the
reference library itself when oracle/_ref/libpulp_ref.so travelled with the repository.
fp32 bar: max|a-b|/max|b| <= 1e-5.  fp16 (storage fp16, accumulation fp32): <= 1e-2 against the
oracle run in fp32 on the fp16-rounded inputs.  Index helpers: bit-exact."""
import os

import numpy as np
import pytest

import golden_cases
from abi_runner import AbiRunner
from metrics import FP16_TOL, FP32_TOL, assert_close, assert_exact, rel_err, seeded
from oracle_bind import geom, out_hw
from test_golden_cpu import load_case

pytestmark = pytest.mark.gpu
F = np.float32


@pytest.fixture()
def run(pkg, gpulib):
    rs = []

    def make(device=False, half=False):
        gpulib.trainlib_set_streams(1)
        r = AbiRunner(pkg, gpulib, device=device, half=half)
        rs.append(r)
        return r
    yield make
    for r in rs:
        r.close()
    gpulib.trainlib_set_streams(1)


@pytest.mark.parametrize("name", [c[0] for c in golden_cases.CASES])
def test_golden_vectors(run, oracle, gpulib, name):
    _, _, run_abi, run_oracle, tol = next(c for c in golden_cases.CASES if c[0] == name)
    inp, want = load_case(name)
    got_host = run_abi(run(device=False), inp)
    got_dev = run_abi(run(device=True), inp)
    orc = run_oracle(oracle, inp)
    for k, v in want.items():
        for mode, got in (("host-pointer", got_host), ("device-pointer", got_dev)):
            g = np.asarray(got[k]).reshape(v.shape)
            if tol is None and name == "index_helpers":
                assert_exact(g.astype(v.dtype), v, "%s.%s (%s mode)" % (name, k, mode))
            else:
                assert_close(g, v, FP32_TOL, "%s.%s vs reference golden (%s mode)" % (name, k, mode))
                assert_close(g, np.asarray(orc[k]).reshape(v.shape), FP32_TOL, "%s.%s vs oracle (%s mode)" % (name, k, mode))
    # The two memory modes run the same kernels on the same values: with the fixed-order FFMA kernels the results are
    # bit-identical (the tensor-core convolution adds in an order that varies from run to run, so it is pinned off here).
    gpulib.trainlib_set_gemm_path(1)
    try:
        h2, d2 = run_abi(run(device=False), inp), run_abi(run(device=True), inp)
    finally:
        gpulib.trainlib_set_gemm_path(0)
    for k, v in want.items():
        assert_exact(np.asarray(d2[k]).reshape(v.shape), np.asarray(h2[k]).reshape(v.shape), "%s.%s device-pointer mode vs host-pointer mode" % (name, k))


def test_torch_golden_model_of_mhsa(run):
    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "mhsa_torch_gm.npz"))
    L, E, Fd, heads = int(z["L"]), int(z["E"]), int(z["F"]), int(z["heads"])
    r = run().mhsa(z["in_x"], z["in_wq"], z["in_wk"], z["in_wv"], z["in_bq"], z["in_bk"], z["in_bv"], z["in_wo"], z["in_dy"], L, E, Fd, heads)
    for k in ("y", "dx", "dwq", "dwk", "dwv", "dwo"):
        assert_close(r[k], z["out_" + k], FP32_TOL, "mhsa vs torch gm %s" % k)


@pytest.mark.parametrize("trans_B", [0, 1])
def test_mm_small_shape_sweep(run, oracle, trans_B):
    """every N, M, K in a set with odd leftovers, incl. K=1, M=1, N=1"""
    rng = seeded(99 + trans_B)
    r = run(device=True)
    dims = (1, 2, 3, 5, 8, 17, 33, 65)
    worst = 0.0
    for N in dims:
        for K in dims:
            for M in dims:
                A = rng.standard_normal((N, K)).astype(F)
                B = rng.standard_normal((M, K) if trans_B else (K, M)).astype(F)
                e = rel_err(r.mm(A, B, N, K, M, trans_B), oracle.mm(A, B, N, K, M, trans_B))
                worst = max(worst, e)
                assert e <= FP32_TOL, (N, K, M, e)
        r.close()


@pytest.mark.parametrize("N,K,M", [(32, 144, 1024), (32, 1024, 144), (16, 288, 1024), (256, 256, 256), (300, 700, 130)])
def test_mm_config_shapes(run, oracle, N, K, M):
    rng = seeded(N + K + M)
    A = rng.standard_normal((N, K)).astype(F); B = rng.standard_normal((K, M)).astype(F); Bt = np.ascontiguousarray(B.T)
    r = run(device=True)
    want = oracle.mm(A, B, N, K, M, 0)
    assert_close(r.mm(A, B, N, K, M, 0), want, FP32_TOL, "mm")
    assert_close(r.mm(A, Bt, N, K, M, 1, fn="mm_unroll_2x4"), want, FP32_TOL, "mm trans_B")
    C0 = rng.standard_normal((N, M)).astype(F)
    assert_close(r.mm(A, B, N, K, M, 0, fn="mm_add", C0=C0), want + C0, FP32_TOL, "mm_add")


@pytest.mark.parametrize("path", [2, 3], ids=["staged", "tma"])
@pytest.mark.parametrize("half", [False, True], ids=["fp32_3xtf32", "fp16"])
@pytest.mark.parametrize("N,K,M", [(128, 64, 128), (130, 70, 67), (1, 1, 1), (257, 33, 129), (64, 512, 200), (384, 256, 256), (5, 1000, 3), (300, 264, 520)])
def test_mm_tensor_core_path(pkg, gpulib, run, oracle, N, K, M, half, path):
    """tcgen05 GEMMs forced on for every shape (tails in all three dimensions, both B layouts, accumulate form):
    path 2 = operands staged by threads, path 3 = TMA-fed (operands packed K-major where needed)"""
    rng = seeded(7 * N + 3 * K + M + (1 if half else 0))
    A = rng.standard_normal((N, K)).astype(F); B = rng.standard_normal((K, M)).astype(F)
    C0 = rng.standard_normal((N, M)).astype(F)
    if half:
        A, B, C0 = [a.astype(np.float16).astype(F) for a in (A, B, C0)]
    Bt = np.ascontiguousarray(B.T)
    tol = FP16_TOL if half else FP32_TOL
    want = oracle.mm(A, B, N, K, M, 0)
    gpulib.trainlib_set_gemm_path(path)
    try:
        r = run(device=True, half=half)
        l0 = gpulib.trainlib_kernel_launches()
        assert_close(r.mm(A, B, N, K, M, 0).astype(F), want, tol, "mm")
        assert gpulib.trainlib_kernel_launches() >= l0 + 1
        assert_close(r.mm(A, Bt, N, K, M, 1).astype(F), want, tol, "mm trans_B")
        if not half:
            assert_close(r.mm(A, B, N, K, M, 0, fn="mm_add", C0=C0), want + C0, tol, "mm_add")
        assert gpulib.trainlib_tc_status() == 0, "a bounded tensor-core wait gave up: id %d" % gpulib.trainlib_tc_status()
    finally:
        gpulib.trainlib_set_gemm_path(0)


@pytest.mark.parametrize("inn,out", [(256, 256), (1024, 1024), (4096, 1024), (1024, 4096), (1000, 37)])
@pytest.mark.parametrize("half", [False, True])
def test_linear_config2(run, oracle, inn, out, half):
    """config 2: W ~ N(0, 1/in), x ~ N(0,1), dy ~ N(0,1); FW, WG, IG"""
    rng = seeded(inn * 3 + out)
    W = (rng.standard_normal((out, inn)) / np.sqrt(inn)).astype(F); x = rng.standard_normal(inn).astype(F); dy = rng.standard_normal(out).astype(F)
    bias = rng.standard_normal(out).astype(F)
    if half:
        W, x, dy, bias = [a.astype(np.float16).astype(F) for a in (W, x, dy, bias)]
    want = oracle.linear(W, x, dy, bias)
    got = run(device=True, half=half).linear(W, x, dy, bias)
    tol = FP16_TOL if half else FP32_TOL
    for k in ("y", "dW", "dx", "db"):
        assert_close(got[k].astype(F).reshape(want[k].shape), want[k], tol, "linear %s" % k)


@pytest.mark.parametrize("half", [False, True])
@pytest.mark.parametrize("inn,out,device", [(256, 256, True), (1024, 4096, True), (4096, 1024, True), (1024, 1000, False), (8, 3, True), (100, 37, True), (4104, 9, True)])
def test_linear_backward_in_one_call(pkg, gpulib, run, oracle, inn, out, device, half):
    """pulp_linear_*_bw_cl with both gradients wanted: one fused launch where the rows are whole 16-byte strips (the kernel
    name proves it), the two separate kernels otherwise; device-resident and host buffers; against the reference and
    bit-identical, launch after launch, with itself"""
    rng = seeded(inn + 5 * out)
    W = (rng.standard_normal((out, inn)) / np.sqrt(inn)).astype(F); x = rng.standard_normal(inn).astype(F); dy = rng.standard_normal(out).astype(F)
    bias = rng.standard_normal(out).astype(F)
    if half:
        W, x, dy, bias = [a.astype(np.float16).astype(F) for a in (W, x, dy, bias)]
    want = oracle.linear(W, x, dy, bias)
    gpulib.trainlib_profile(1)
    got = run(device=device, half=half).linear(W, x, dy, bias, one_backward_call=True)
    gpulib.trainlib_profile(0)
    names = [row[0] for row in pkg.profile_table(gpulib)]
    assert any("linear_bw_fused_kernel" in nm for nm in names) == (inn % (8 if half else 4) == 0), names
    tol = FP16_TOL if half else FP32_TOL
    for k in ("y", "dW", "dx", "db"):
        assert_close(got[k].astype(F).reshape(want[k].shape), want[k], tol, "linear %s" % k)
    again = run(device=device, half=half).linear(W, x, dy, bias, one_backward_call=True)
    for k in ("dW", "dx"):
        assert np.array_equal(got[k], again[k]), "fused linear backward is not reproducible: %s" % k


CONV_CASES = [geom(16, 32, 32, 32, 3, pad=1), geom(3, 32, 32, 16, 3, pad=1), geom(16, 32, 32, 32, 3, stride=2, pad=1),
              geom(32, 16, 16, 64, 3, stride=2, pad=1), geom(64, 8, 8, 64, 3, pad=1), geom(16, 32, 32, 32, 1, stride=2),
              geom(5, 11, 13, 7, 3, stride=2, pad=1), geom(3, 9, 9, 4, 5, stride=1, pad=2), geom(2, 12, 12, 3, 7, pad=3),
              geom(1, 5, 5, 1, 3), geom(20, 6, 6, 33, 3, pad=1), geom(4, 8, 8, 4, 2)]


@pytest.mark.parametrize("g", CONV_CASES, ids=lambda g: "c%d_%dx%d_o%d_k%d_s%d_p%d" % (g["Cin"], g["Hin"], g["Win"], g["Cout"], g["Hk"], g["sh"], g["padU"]))
@pytest.mark.parametrize("half", [False, True])
def test_conv2d_sweep(run, oracle, g, half):
    rng = seeded(g["Cin"] * 31 + g["Hin"] + g["Hk"])
    Ho, Wo = out_hw(g)
    x = rng.uniform(-1, 1, (g["Cin"], g["Hin"], g["Win"])).astype(F)
    w = rng.uniform(-1, 1, (g["Cout"], g["Cin"], g["Hk"], g["Wk"])).astype(F)
    dy = rng.standard_normal((g["Cout"], Ho, Wo)).astype(F); bias = rng.standard_normal(g["Cout"]).astype(F)
    if half:
        x, w, dy, bias = [a.astype(np.float16).astype(F) for a in (x, w, dy, bias)]
    got = run(device=True, half=half).conv2d(x, w, dy, g, use_im2col=0, bias=bias)
    tol = FP16_TOL if half else FP32_TOL
    assert_close(got["y"].astype(F), oracle.conv2d_fw(x, w, bias, g), tol, "fw")
    dw, db = oracle.conv2d_wg(x, dy, g, with_bias=True)
    assert_close(got["dw"].astype(F), dw, tol, "wg")
    assert_close(got["db"].astype(F), db, tol, "bias grad")
    assert_close(got["dx"].astype(F), oracle.conv2d_ig(dy, w, g), tol, "ig")


TC_CASES = [(geom(16, 32, 32, 16, 3, pad=1), 2), (geom(16, 32, 32, 32, 3, stride=2, pad=1), 3), (geom(32, 16, 16, 32, 3, pad=1), 1),
            (geom(32, 16, 16, 64, 3, stride=2, pad=1), 2), (geom(64, 8, 8, 64, 3, pad=1), 3), (geom(16, 32, 32, 32, 1, stride=2), 2),
            (geom(3, 32, 32, 16, 3, pad=1), 2), (geom(20, 64, 64, 40, 3, pad=1), 1), (geom(16, 32, 32, 16, 5, pad=2), 1),
            (geom(16, 32, 32, 16, 3, stride=2, pad=0), 2), (geom(32, 16, 16, 64, 1, stride=2), 5)]


@pytest.mark.parametrize("g,n", TC_CASES, ids=lambda v: str(v) if isinstance(v, int) else "c%d_%d_o%d_k%d_s%d" % (v["Cin"], v["Hin"], v["Cout"], v["Hk"], v["sh"]))
def test_conv2d_tensor_core_path(pkg, gpulib, oracle, g, n):
    """tcgen05 implicit-GEMM kernels (3xTF32) forced on, n streams per launch, against the fp32 oracle"""
    rng = seeded(g["Cin"] + 7 * g["Cout"] + n)
    Ho, Wo = out_hw(g)
    xs = rng.uniform(-1, 1, (n, g["Cin"], g["Hin"], g["Win"])).astype(F); w = rng.uniform(-1, 1, (g["Cout"], g["Cin"], g["Hk"], g["Wk"])).astype(F)
    dys = rng.standard_normal((n, g["Cout"], Ho, Wo)).astype(F)
    gpulib.trainlib_set_streams(n); gpulib.trainlib_set_gemm_path(2)
    try:
        r = AbiRunner(pkg, gpulib, device=True)
        X, W_, dY = r.t(xs), r.t(w), r.t(dys)
        Y, dX, dW, one = r.zeros(n, g["Cout"], Ho, Wo), r.zeros(*xs.shape), r.zeros(*w.shape), r.zeros(1)
        args = r.args("Conv2D_args", input=r.blob(X, dX, C=g["Cin"], H=g["Hin"], W=g["Win"]), coeff=r.blob(W_, dW, C=g["Cin"], H=g["Hk"], W=g["Wk"], dim=w.size),
                      bias=r.blob(one, one), output=r.blob(Y, dY, C=g["Cout"], H=Ho, W=Wo), Lpad=g["padL"], Rpad=g["padR"], Upad=g["padU"], Dpad=g["padD"],
                      stride_h=g["sh"], stride_w=g["sw"], i2c_buffer=one, bt_buffer=one, USE_BIASES=0, USE_IM2COL=1, HWC=0)
        l0 = gpulib.trainlib_kernel_launches()
        r.call("pulp_conv2d_fp32_fw_cl", args); r.call("pulp_conv2d_fp32_bw_input_grads_cl", args)
        assert gpulib.trainlib_tc_status() == 0, "a bounded tensor-core wait gave up: id %d" % gpulib.trainlib_tc_status()
        y, dx = Y.get(), dX.get()
        for s in range(n):
            assert_close(y[s], oracle.conv2d_fw(xs[s], w, None, g), FP32_TOL, "tc fw stream %d" % s)
            assert_close(dx[s], oracle.conv2d_ig(dys[s], w, g), FP32_TOL, "tc ig stream %d" % s)
        # the weight gradient (sum over the streams); 3x3 / pad 1 layers with stride 1 or 2 and channel counts in multiples of
        # 8 / 16 go through the tensor-core pixel-contraction kernel when forced, which the kernel names prove
        gpulib.trainlib_profile(1)
        r.call("pulp_conv2d_fp32_bw_param_grads_cl", args)
        gpulib.trainlib_profile(0)
        assert gpulib.trainlib_tc_status() == 0, "a bounded tensor-core wait gave up: id %d" % gpulib.trainlib_tc_status()
        names = [row[0] for row in pkg.profile_table(gpulib)]
        eligible = (g["Hk"] == 3 and g["padU"] == 1 and g["Cin"] % 8 == 0 and g["Cout"] % 16 == 0 and g["Cin"] <= 64 and g["Cout"] <= 64
                    and Wo in (8, 16, 32) and not (g["sh"] == 2 and Wo == 32))
        assert any("conv_wgt_kernel" in nm for nm in names) == eligible, (names, eligible)
        want = sum(oracle.conv2d_wg(xs[s], dys[s], g)[0].astype(np.float64) for s in range(n)).astype(F)
        assert_close(dW.get(), want, FP32_TOL, "tc weight gradient")
        r.close()
    finally:
        gpulib.trainlib_set_streams(1); gpulib.trainlib_set_gemm_path(0)


C1_CASES = [(geom(16, 32, 32, 32, 1, stride=2), 5), (geom(32, 16, 16, 64, 1, stride=2), 3), (geom(8, 18, 18, 12, 1, stride=3), 2),
            (geom(64, 10, 10, 64, 1, stride=2), 300), (geom(4, 33, 33, 4, 1, stride=2), 1), (geom(16, 17, 17, 16, 1, stride=2), 7),
            (geom(32, 20, 20, 32, 1, stride=3), 4), (geom(64, 8, 8, 128, 1, stride=2), 2), (geom(32, 64, 64, 16, 1, stride=2), 2)]


@pytest.mark.parametrize("g,n", C1_CASES, ids=lambda v: str(v) if isinstance(v, int) else "c%d_%d_o%d_s%d" % (v["Cin"], v["Hin"], v["Cout"], v["sh"]))
def test_conv2d_1x1_strided_kernels(pkg, gpulib, oracle, g, n):
    """projection shortcuts (1x1, stride > 1, no padding) at the default dispatch: forward with bias, weight gradient summed
    over the streams, input gradient stored and added in place; pixel counts that are not multiples of the tile included"""
    rng = seeded(5 * g["Cin"] + g["Cout"] + n)
    Ho, Wo = out_hw(g)
    xs = rng.uniform(-1, 1, (n, g["Cin"], g["Hin"], g["Win"])).astype(F); w = rng.uniform(-1, 1, (g["Cout"], g["Cin"], 1, 1)).astype(F)
    b = rng.uniform(-1, 1, g["Cout"]).astype(F); dys = rng.standard_normal((n, g["Cout"], Ho, Wo)).astype(F)
    base = rng.uniform(-1, 1, xs.shape).astype(F)
    gpulib.trainlib_set_streams(n)
    try:
        r = AbiRunner(pkg, gpulib, device=True)
        X, W_, B, dY = r.t(xs), r.t(w), r.t(b), r.t(dys)
        Y, dX, dW, dB, one = r.zeros(n, g["Cout"], Ho, Wo), r.t(base), r.zeros(*w.shape), r.zeros(g["Cout"]), r.zeros(1)
        args = r.args("Conv2D_args", input=r.blob(X, dX, C=g["Cin"], H=g["Hin"], W=g["Win"]), coeff=r.blob(W_, dW, C=g["Cin"], H=1, W=1, dim=w.size),
                      bias=r.blob(B, dB, dim=g["Cout"]), output=r.blob(Y, dY, C=g["Cout"], H=Ho, W=Wo), Lpad=0, Rpad=0, Upad=0, Dpad=0,
                      stride_h=g["sh"], stride_w=g["sw"], i2c_buffer=one, bt_buffer=one, USE_BIASES=1, USE_IM2COL=1, HWC=0)
        gpulib.trainlib_profile(1)
        r.call("pulp_conv2d_fp32_fw_cl", args); r.call("pulp_conv2d_fp32_bw_param_grads_cl", args)
        r.call("trainlib_conv2d_fp32_bw_input_grads_acc_cl", args)
        gpulib.trainlib_profile(0)
        names = [row[0] for row in pkg.profile_table(gpulib)]
        # channel counts in multiples of 16 run on the dedicated kernels (the contraction of the input gradient up to 64)
        if g["Cin"] % 16 == 0 and g["Cout"] % 16 == 0:
            want_names = ["conv1x1s_mma_kernel<%d, " % (g["Cin"] // 8), "conv1x1s_wg_kernel"] + (["conv1x1s_mma_kernel<%d, " % (g["Cout"] // 8)] if g["Cout"] <= 64 else [])
            for k in want_names:
                assert any(k in nm for nm in names), (k, names)
        y, dx_acc = Y.get(), dX.get()
        r.call("pulp_conv2d_fp32_bw_input_grads_cl", args)
        dx = dX.get()
        for s in sorted({0, n // 2, n - 1}):
            assert_close(y[s], oracle.conv2d_fw(xs[s], w, b, g), FP32_TOL, "1x1 fw stream %d" % s)
            ig = oracle.conv2d_ig(dys[s], w, g)
            assert_close(dx[s], ig, FP32_TOL, "1x1 ig stream %d" % s)
            assert_close(dx_acc[s], (base[s].astype(np.float64) + ig).astype(F), FP32_TOL, "1x1 ig added in place, stream %d" % s)
        want = sum(oracle.conv2d_wg(xs[s], dys[s], g)[0].astype(np.float64) for s in range(n)).astype(F)
        assert_close(dW.get(), want, FP32_TOL, "1x1 weight gradient")
        assert_close(dB.get(), dys.astype(np.float64).sum(axis=(0, 2, 3)).astype(F), FP32_TOL, "1x1 bias gradient")
        r.close()
    finally:
        gpulib.trainlib_set_streams(1)


def test_conv2d_tensor_core_many_tiles(pkg, gpulib, oracle):
    """long persistent loops (hundreds of tiles per CTA): every barrier ring wraps many times; a few streams are checked"""
    g = geom(16, 32, 32, 16, 3, pad=1)
    n = 3000
    rng = seeded(77)
    xs = rng.uniform(-1, 1, (n, 16, 32, 32)).astype(F); w = rng.uniform(-1, 1, (16, 16, 3, 3)).astype(F)
    gpulib.trainlib_set_streams(n)
    try:
        r = AbiRunner(pkg, gpulib, device=True)
        X, W_ = r.t(xs), r.t(w)
        Y, one = r.zeros(n, 16, 32, 32), r.zeros(1)
        args = r.args("Conv2D_args", input=r.blob(X, one, C=16, H=32, W=32), coeff=r.blob(W_, one, C=16, H=3, W=3, dim=w.size), bias=r.blob(one, one),
                      output=r.blob(Y, one, C=16, H=32, W=32), Lpad=1, Rpad=1, Upad=1, Dpad=1, stride_h=1, stride_w=1, i2c_buffer=one, bt_buffer=one,
                      USE_BIASES=0, USE_IM2COL=1, HWC=0)
        r.call("pulp_conv2d_fp32_fw_cl", args)
        assert gpulib.trainlib_tc_status() == 0, "a bounded tensor-core wait gave up: id %d" % gpulib.trainlib_tc_status()
        y = Y.get()
        for s in (0, 1, 147, 148, 1499, 2998, 2999):
            assert_close(y[s], oracle.conv2d_fw(xs[s], w, None, g), FP32_TOL, "stream %d" % s)
        r.close()
    finally:
        gpulib.trainlib_set_streams(1)


def test_mhsa_config3(run, oracle):
    """config 3: L = E = F = 256, 4 heads of 64; x ~ N(0,1), W ~ N(0, 1/E), dy ~ N(0,1), zero biases"""
    rng = seeded(3)
    L = E = Fd = 256; heads = 4
    x = rng.standard_normal((E, L)).astype(F); dy = rng.standard_normal((E, L)).astype(F)
    ws = [(rng.standard_normal((E, Fd)) / np.sqrt(E)).astype(F) for _ in range(4)]
    zb = np.zeros(Fd, F)
    want = oracle.mhsa(x, ws[0], ws[1], ws[2], zb, zb, zb, ws[3], dy, L, E, Fd, heads)
    got = run(device=True).mhsa(x, ws[0], ws[1], ws[2], zb, zb, zb, ws[3], dy, L, E, Fd, heads)
    for k in ("q", "k", "v", "softmax", "att", "y", "dwo", "datt", "dv", "dsoftmax", "dk", "dq", "dwq", "dwk", "dwv", "dx"):
        assert_close(got[k], want[k], FP32_TOL, "mhsa c3 %s" % k)


@pytest.mark.parametrize("L,E,Fd,heads", [(37, 24, 36, 3), (100, 48, 80, 2), (256, 64, 128, 4), (8, 16, 16, 1), (1, 8, 8, 2)])
def test_mhsa_fused_attention_core(run, pkg, gpulib, oracle, L, E, Fd, heads):
    """ragged sequence lengths and head sizes through the fused score-softmax-value kernels; the same call with the fused
    kernels switched off (gemm path 1) must agree too, and the kernel names prove which path ran"""
    rng = seeded(31 + L)
    x = rng.standard_normal((E, L)).astype(F); dy = rng.standard_normal((E, L)).astype(F)
    ws = [(rng.standard_normal((E, Fd)) / np.sqrt(E)).astype(F) for _ in range(3)] + [(rng.standard_normal((E, Fd)) / np.sqrt(Fd)).astype(F)]
    bs = [(0.1 * rng.standard_normal(Fd)).astype(F) for _ in range(3)]
    want = oracle.mhsa(x, ws[0], ws[1], ws[2], bs[0], bs[1], bs[2], ws[3], dy, L, E, Fd, heads)
    gpulib.trainlib_profile(1)
    got = run(device=True).mhsa(x, ws[0], ws[1], ws[2], bs[0], bs[1], bs[2], ws[3], dy, L, E, Fd, heads)
    gpulib.trainlib_profile(0)
    names = [r[0] for r in pkg.profile_table(gpulib)]
    for kernel in ("attn_fw_kernel", "attn_bw_query_kernel", "attn_bw_key_kernel"):
        assert any(kernel in n for n in names), "%s did not run: %s" % (kernel, names)
    assert not any("softmax" in n for n in names), "the separate softmax kernels ran beside the fused ones: %s" % names
    try:
        gpulib.trainlib_set_gemm_path(1)
        plain = run(device=True).mhsa(x, ws[0], ws[1], ws[2], bs[0], bs[1], bs[2], ws[3], dy, L, E, Fd, heads)
    finally:
        gpulib.trainlib_set_gemm_path(0)
    for k in ("q", "k", "v", "softmax", "att", "y", "dwo", "datt", "dv", "dsoftmax", "dk", "dq", "dwq", "dwk", "dwv", "dx"):
        assert_close(got[k], want[k], FP32_TOL, "fused mhsa %s" % k)
        assert_close(plain[k], want[k], FP32_TOL, "unfused mhsa %s" % k)


def _mobilebert_inputs(rng, L, E, Kb, Fd, No, cast=lambda a: a):
    f = lambda *s: rng.standard_normal(s).astype(F)
    d = dict(x=f(L, E), xb=f(L, Kb), dy=f(L, No), wq=f(Fd, Kb) / np.sqrt(Kb), wk=f(Fd, Kb) / np.sqrt(Kb), wv=f(Fd, E) / np.sqrt(E),
             wo=f(No, Fd) / np.sqrt(Fd), bq=0.1 * f(Fd), bk=0.1 * f(Fd), bv=0.1 * f(Fd), bo=0.1 * f(No))
    return {k: cast(v.astype(F)) for k, v in d.items()}


MB_KEYS = ("q", "k", "v", "softmax", "att", "y", "dwo", "datt", "dv", "dsoftmax", "dk", "dq", "dwq", "dwk", "dwv", "dx", "dxb")


@pytest.mark.parametrize("L,E,Fd,heads", [(24, 20, 32, 4), (128, 512, 128, 4), (37, 48, 40, 5)])
def test_mobilebert_attention_forward_backward(run, oracle, L, E, Fd, heads):
    """pulp_mhsa_mobilebert_inference_fp32_{fw,bw}_cl (F = Kb = No) against the oracle; the middle case is the attention
    of config 4's block (sequence 128, hidden 512, bottleneck 128, 4 heads of 32)"""
    i = _mobilebert_inputs(seeded(L + E), L, E, Fd, Fd, Fd)
    a = (i["x"], i["xb"], i["wq"], i["wk"], i["wv"], i["bq"], i["bk"], i["bv"], i["wo"], i["bo"], i["dy"], L, E, Fd, Fd, Fd, heads)
    want = oracle.mobilebert(*a)
    got = run(device=True).mobilebert(*a)
    for k in MB_KEYS:
        assert_close(got[k], want[k], FP32_TOL, "mobilebert attention %s" % k)
    # host pointers (staging mirrors) give the same bits as device pointers
    host = run(device=False).mobilebert(*a)
    for k in MB_KEYS:
        assert_exact(host[k], got[k], "mobilebert attention, host pointers, %s" % k)


def test_mobilebert_attention_input_gradients_into_one_buffer(run, oracle):
    """input_bn without a diff buffer and Kb = E: all three input gradients are added into input.diff, as the reference does"""
    L, E, heads = 16, 24, 3
    i = _mobilebert_inputs(seeded(8), L, E, E, E, E)
    a = (i["x"], i["xb"], i["wq"], i["wk"], i["wv"], i["bq"], i["bk"], i["bv"], i["wo"], i["bo"], i["dy"], L, E, E, E, E, heads)
    want = oracle.mobilebert(*a)
    got = run(device=True).mobilebert(*a, share_input_diff=True)
    assert_close(got["dx"], want["dx"] + want["dxb"], FP32_TOL, "summed input gradient")


def test_tiled_mhsa_sizes_from_the_coefficient_blobs(run, oracle):
    """tiled_mhsa_fp32: F, Kb and No come from the coefficient blobs and differ from one another; tile sizes are ignored"""
    L, E, Kb, Fd, No, heads = 40, 36, 28, 48, 20, 6
    i = _mobilebert_inputs(seeded(9), L, E, Kb, Fd, No)
    a = (i["x"], i["xb"], i["wq"], i["wk"], i["wv"], i["bq"], i["bk"], i["bv"], i["wo"], i["bo"], None, L, E, Kb, Fd, No, heads)
    want = oracle.mobilebert(*a)
    got = run(device=True).mobilebert(*a, tiled=True)
    for k in ("q", "k", "v", "softmax", "att", "y"):
        assert_close(got[k], want[k], FP32_TOL, "tiled attention %s" % k)


def test_tiled_matmul_and_transpose_mhsa(pkg, gpulib, oracle):
    rng = seeded(10)
    N, K, M = 24, 16, 40
    A = rng.standard_normal((N, K)).astype(F); B = rng.standard_normal((M, K)).astype(F); bias = rng.standard_normal(N).astype(F)
    r = AbiRunner(pkg, gpulib, device=True)
    a, b, c, bi = r.t(A), r.t(B), r.zeros(N, M), r.t(bias)
    args = r.args("matMul_args", A=a, B=b, C=c, N=N, K=K, M=M, trans_B=1, USE_BIASES=1, bias=bi, bias_transposed=1, bias_dim=N)
    targs = r.args("Tiled_Matmul_Mhsa_args", tile_h=8, tile_w=8, tile_dim=64)
    import ctypes
    gpulib.tiled_matmul_mhsa(ctypes.byref(args), ctypes.byref(targs), 1); pkg.check(gpulib)
    want = oracle.mm(A, B, N, K, M, 1) + bias[:, None]
    assert_close(c.get(), want, FP32_TOL, "tiled_matmul_mhsa")
    out = r.zeros(M, N)
    targ = r.args("transp_args", in_matrix=c, out_matrix=out, N=N, M=M)
    gpulib.tiled_transpose_mhsa(ctypes.byref(targ), ctypes.byref(targs), 0); pkg.check(gpulib)
    assert_exact(out.get(), c.get().T, "tiled_transpose_mhsa")
    r.close()


def test_mobilebert_attention_fp16(run, oracle):
    """fp16 twins (inference forward / backward and tiled forward) against the fp32 oracle on fp16-representable inputs"""
    L, E, Fd, heads = 128, 512, 128, 4
    h = lambda a: a.astype(np.float16).astype(F)
    i = _mobilebert_inputs(seeded(12), L, E, Fd, Fd, Fd, cast=h)
    a = (i["x"], i["xb"], i["wq"], i["wk"], i["wv"], i["bq"], i["bk"], i["bv"], i["wo"], i["bo"], i["dy"], L, E, Fd, Fd, Fd, heads)
    want = oracle.mobilebert(*a)
    got = run(device=True, half=True).mobilebert(*a)
    for k in ("y", "softmax", "att", "dx", "dxb", "dwq", "dwk", "dwv", "dwo"):
        assert_close(got[k].astype(F), want[k], 2e-2, "mobilebert attention fp16 %s" % k)     # intermediates are rounded to fp16 between the kernels
    tiled = run(device=True, half=True).mobilebert(*(a[:10] + (None,) + a[11:]), tiled=True)
    assert_exact(tiled["y"], got["y"], "tiled_mhsa_fp16 = inference forward on square shapes")


def test_mhsa_fp16(run, oracle):
    rng = seeded(4)
    L, E, Fd, heads = 128, 128, 128, 4
    h = lambda a: a.astype(np.float16).astype(F)
    x = h(rng.standard_normal((E, L))); dy = h(rng.standard_normal((E, L)))
    ws = [h(rng.standard_normal((E, Fd)) / np.sqrt(E)) for _ in range(4)]
    bs = [h(0.1 * rng.standard_normal(Fd)) for _ in range(3)]
    want = oracle.mhsa(x, ws[0], ws[1], ws[2], bs[0], bs[1], bs[2], ws[3], dy, L, E, Fd, heads)
    got = run(device=True, half=True).mhsa(x, ws[0], ws[1], ws[2], bs[0], bs[1], bs[2], ws[3], dy, L, E, Fd, heads)
    for k in ("y", "softmax", "dx", "dwq", "dwk", "dwv", "dwo"):
        assert_close(got[k].astype(F), want[k], 2e-2, "mhsa fp16 %s" % k)     # intermediates are rounded to fp16 between the GEMMs


def test_fp16_elementwise(run, oracle):
    rng = seeded(5)
    h = lambda a: a.astype(np.float16).astype(F)
    x = h(2 * rng.standard_normal(4096)); dy = h(rng.standard_normal(4096))
    r = run(device=True, half=True)
    for k, kind in enumerate(("relu", "leakyrelu", "sigmoid")):
        res = r.act(kind, x, dy, slope=0.01)
        y = oracle.act_fw(k, x, h(np.array([0.01]))[0])
        assert_close(res["y"].astype(F), y, FP16_TOL, kind)
        assert_close(res["dx"].astype(F), oracle.act_bw(k, x, y, dy, h(np.array([0.01]))[0]), FP16_TOL, kind + " bw")
    assert_close(r.act("gelu", x, dy)["y"].astype(F), oracle.act_fw(3, x), FP16_TOL, "gelu")
    xi = h(rng.standard_normal((8, 16, 16))); dyi = h(rng.standard_normal((8, 16, 16))); gb = h(rng.standard_normal(16))
    res = r.instnorm(xi, gb, dyi); want = oracle.instnorm(xi, gb, dyi)
    for k in ("y", "dx", "dgb"):
        assert_close(res[k].astype(F), want[k], FP16_TOL, "instnorm fp16 %s" % k)
    y = h(rng.standard_normal(512)); t = h(rng.standard_normal(512))
    loss, dyl = r.loss("MSELoss", y, t); lo, dyo = oracle.mse(y, t)
    assert abs(float(loss) - float(lo)) <= FP16_TOL * abs(float(lo)); assert_close(dyl.astype(F), dyo, FP16_TOL, "mse bw fp16")
    s = r.sgd(x, dy, 0.01); wo, _ = oracle.sgd(x, dy, h(np.array([0.01]))[0])
    assert_close(s["w"].astype(F), wo, FP16_TOL, "sgd fp16")


def test_streams_mode(pkg, gpulib, oracle):
    """n independent batch-1 streams in one call: activations per stream, weight gradients summed."""
    rng = seeded(6)
    n = 5
    g = geom(6, 12, 12, 10, 3, pad=1)
    Ho, Wo = out_hw(g)
    xs = rng.uniform(-1, 1, (n, 6, 12, 12)).astype(F); w = rng.uniform(-1, 1, (10, 6, 3, 3)).astype(F); dys = rng.standard_normal((n, 10, Ho, Wo)).astype(F)
    gpulib.trainlib_set_streams(n)
    try:
        r = AbiRunner(pkg, gpulib, device=True)
        # the runner's blobs describe one stream; the tensors hold n of them back to back
        X, W_, dY = r.t(xs), r.t(w), r.t(dys)
        Y, dX, dW = r.zeros(n, 10, Ho, Wo), r.zeros(n, 6, 12, 12), r.zeros(10, 6, 3, 3)
        one = r.zeros(1)
        args = r.args("Conv2D_args", input=r.blob(X, dX, C=6, H=12, W=12), coeff=r.blob(W_, dW, C=6, H=3, W=3, dim=w.size), bias=r.blob(one, one),
                      output=r.blob(Y, dY, C=10, H=Ho, W=Wo), Lpad=1, Rpad=1, Upad=1, Dpad=1, stride_h=1, stride_w=1, i2c_buffer=one, bt_buffer=one,
                      USE_BIASES=0, USE_IM2COL=1, HWC=0)
        r.call("pulp_conv2d_fp32_fw_cl", args); r.call("pulp_conv2d_fp32_bw_cl", args)
        y, dx, dw = Y.get(), dX.get(), dW.get()
        dw_want = np.zeros_like(w)
        for s in range(n):
            assert_close(y[s], oracle.conv2d_fw(xs[s], w, None, g), FP32_TOL, "stream %d fw" % s)
            assert_close(dx[s], oracle.conv2d_ig(dys[s], w, g), FP32_TOL, "stream %d ig" % s)
            dw_want += oracle.conv2d_wg(xs[s], dys[s], g)[0]
        assert_close(dw, dw_want, FP32_TOL, "summed weight grad")
        # instance norm + relu + CE + linear over streams
        gb = rng.standard_normal(12).astype(F)
        xi = xs; dyi = rng.standard_normal(xs.shape).astype(F)
        Xi, dXi, Yi, dYi, GB, dGB = r.t(xi), r.zeros(*xi.shape), r.zeros(*xi.shape), r.t(dyi), r.t(gb), r.zeros(12)
        m, v, sd = r.zeros(n, 6), r.zeros(n, 6), r.zeros(n, 6)
        a2 = r.args("InstNorm_args", input=r.blob(Xi, dXi, C=6, H=12, W=12), output=r.blob(Yi, dYi, C=6, H=12, W=12), coeff=r.blob(GB, dGB, dim=12, W=12),
                    running_mean=m, running_var=v, running_stdev=sd, freeze_running_params=0, skip_wg_grad=0, skip_in_grad=0)
        r.call("pulp_instnorm_fp32_fw_cl", a2); r.call("pulp_instnorm_fp32_bw_cl", a2)
        dgb_want = np.zeros(12, F)
        for s in range(n):
            o = oracle.instnorm(xi[s], gb, dyi[s])
            assert_close(Yi.get()[s], o["y"], FP32_TOL, "instnorm stream fw"); assert_close(dXi.get()[s], o["dx"], FP32_TOL, "instnorm stream ig")
            dgb_want += o["dgb"]
        assert_close(dGB.get(), dgb_want, FP32_TOL, "instnorm summed param grad")
        Wl = (rng.standard_normal((10, 64)) / 8).astype(F); xl = rng.standard_normal((n, 64)).astype(F); lab = np.zeros((n, 10), F)
        lab[np.arange(n), rng.integers(0, 10, n)] = 1
        res = r.linear(Wl, xl, np.zeros((n, 10), F), n=n)            # forward only matters here
        z = res["y"].reshape(n, 10)
        for s in range(n):
            assert_close(z[s], oracle.linear(Wl, xl[s], np.zeros(10, F))["y"], FP32_TOL, "linear stream fw")
        Z, dZ, T, Ls = r.t(z), r.zeros(n, 10), r.t(lab), r.zeros(n)
        a3 = r.args("loss_args", output=r.blob(Z, dZ, dim=10, W=10), target=T, wr_loss=Ls)
        r.call("pulp_CrossEntropyLoss", a3); r.call("pulp_CrossEntropyLoss_backward", a3)
        for s in range(n):
            lo, dzo = oracle.ce(z[s], lab[s])
            assert abs(Ls.get()[s] - lo) <= 1e-5 * max(1.0, abs(lo)); assert_close(dZ.get()[s], dzo, FP32_TOL, "ce stream bw")
        dzs = dZ.get()
        res = r.linear(Wl, xl, dzs, n=n)
        dW_want = sum(np.outer(dzs[s], xl[s]) for s in range(n))
        assert_close(res["dW"], dW_want, FP32_TOL, "linear summed weight grad")
        for s in range(n):
            assert_close(res["dx"].reshape(n, 64)[s], oracle.linear(Wl, xl[s], dzs[s])["dx"], FP32_TOL, "linear stream ig")
        r.close()
    finally:
        gpulib.trainlib_set_streams(1)


def test_reference_library_side_by_side(pkg, gpulib, reflib):
    """Same structs, same seeded inputs, the reference's own code on the host vs the GPU library."""
    rng = seeded(8)
    g = geom(8, 16, 16, 12, 3, stride=2, pad=1)
    x = rng.uniform(-1, 1, (8, 16, 16)).astype(F); w = rng.uniform(-1, 1, (12, 8, 3, 3)).astype(F); dy = rng.standard_normal((12,) + out_hw(g)).astype(F)
    ref = AbiRunner(pkg, reflib, is_ref=True).conv2d(x, w, dy, g, use_im2col=0)
    got = AbiRunner(pkg, gpulib).conv2d(x, w, dy, g, use_im2col=0)
    for k in ("y", "dw", "dx"):
        assert_close(got[k], ref[k], FP32_TOL, "conv s2p1 %s vs reference" % k)
    L, E, Fd, heads = 48, 32, 64, 4
    xm = rng.standard_normal((E, L)).astype(F); dym = rng.standard_normal((E, L)).astype(F)
    ws = [(rng.standard_normal((E, Fd)) / np.sqrt(E)).astype(F) for _ in range(4)]; bs = [(0.1 * rng.standard_normal(Fd)).astype(F) for _ in range(3)]
    ref = AbiRunner(pkg, reflib, is_ref=True).mhsa(xm, ws[0], ws[1], ws[2], bs[0], bs[1], bs[2], ws[3], dym, L, E, Fd, heads)
    got = AbiRunner(pkg, gpulib).mhsa(xm, ws[0], ws[1], ws[2], bs[0], bs[1], bs[2], ws[3], dym, L, E, Fd, heads)
    for k in ("y", "dx", "dwq", "dwk", "dwv", "dwo"):
        assert_close(got[k], ref[k].reshape(got[k].shape), FP32_TOL, "mhsa %s vs reference" % k)


def test_error_paths(pkg, gpulib):
    """bad arguments latch an error code and leave outputs untouched, as the reference prints and returns"""
    r = AbiRunner(pkg, gpulib)
    x = np.ones((2, 4, 4), F)
    with pytest.raises(RuntimeError):
        r.conv2d(x, np.ones((3, 2, 3, 3), F), None, dict(geom(2, 4, 4, 3, 3), Hk=5, Wk=5))      # kernel larger than the input
    assert gpulib.trainlib_last_error() == 0           # check() cleared it
    keep = pkg.Keep()
    a = pkg.make_args(keep, "mm_manager_args", mm_args=pkg.make_args(keep, "matMul_args", N=1, M=1, K=1), layer_type=1, step_type=0, matmul_type=0)
    pkg.call(gpulib, "mm_manager", a)
    assert gpulib.trainlib_last_error() == 3
    gpulib.trainlib_clear_error()


def test_cuda_graph_replay_matches_direct_calls(pkg, gpulib, run, oracle):
    """a conv forward + weight gradient recorded with trainlib_graph_begin/end and replayed twice gives what the direct calls give"""
    g = geom(16, 32, 32, 32, 3, pad=1)
    rng = seeded(123)
    x = rng.uniform(-1, 1, (16, 32, 32)).astype(F); w = rng.uniform(-1, 1, (32, 16, 3, 3)).astype(F); dy = rng.standard_normal((32, 32, 32)).astype(F)
    r = run(device=True)
    X, W_, dY = r.t(x), r.t(w), r.t(dy)
    Y, dX, dW, one = r.zeros(32, 32, 32), r.zeros(16, 32, 32), r.zeros(32, 16, 3, 3), r.zeros(1)
    args = r.args("Conv2D_args", input=r.blob(X, dX, C=16, H=32, W=32), coeff=r.blob(W_, dW, C=16, H=3, W=3, dim=w.size), bias=r.blob(one, one),
                  output=r.blob(Y, dY, C=32, H=32, W=32), Lpad=1, Rpad=1, Upad=1, Dpad=1, stride_h=1, stride_w=1, i2c_buffer=one, bt_buffer=one,
                  USE_BIASES=0, USE_IM2COL=0, HWC=0)
    r.call("pulp_conv2d_fp32_fw_cl", args); r.call("pulp_conv2d_fp32_bw_param_grads_cl", args)     # warm-up: scratch arena at its final size
    l0 = gpulib.trainlib_kernel_launches()
    assert gpulib.trainlib_graph_begin() == 0
    r.call("pulp_conv2d_fp32_fw_cl", args); r.call("pulp_conv2d_fp32_bw_param_grads_cl", args)
    graph = gpulib.trainlib_graph_end()
    assert graph, gpulib.trainlib_last_error_string()
    assert gpulib.trainlib_kernel_launches() == l0, "recording must not count as running"
    # new inputs at the same addresses: the replay must compute with them
    x2 = rng.uniform(-1, 1, x.shape).astype(F); dy2 = rng.standard_normal(dy.shape).astype(F)
    X.set(x2); dY.set(dy2)
    for _ in range(2):
        assert gpulib.trainlib_graph_launch(graph) == 0
    recorded = gpulib.trainlib_kernel_launches() - l0
    assert recorded >= 4 and recorded % 2 == 0
    assert_close(Y.get(), oracle.conv2d_fw(x2, w, None, g), FP32_TOL, "graph fw")
    assert_close(dW.get(), oracle.conv2d_wg(x2, dy2, g)[0], FP32_TOL, "graph wg")
    gpulib.trainlib_graph_destroy(graph)


@pytest.mark.parametrize("half", [False, True], ids=["fp32", "fp16"])
@pytest.mark.parametrize("rows,width", [(128, 128), (128, 512), (7, 33)])
def test_layernorm_forward_backward_extension(run, oracle, rows, width, half):
    """layer norm forward (fp16 twin) and backward, which the reference lacks, against the oracle's derivative of the reference formula"""
    rng = seeded(rows + width)
    x = rng.standard_normal((rows, width)).astype(F); w = rng.standard_normal(width).astype(F); b = rng.standard_normal(width).astype(F)
    dy = rng.standard_normal((rows, width)).astype(F)
    if half:
        x, w, b, dy = [a.astype(np.float16).astype(F) for a in (x, w, b, dy)]
    eps = 1e-3 if half else 1e-5
    if half:
        eps = float(np.float16(eps))
    got = run(device=True, half=half).layernorm_ext(x, w, b, dy, rows, width, eps)
    tol = FP16_TOL if half else FP32_TOL
    assert_close(got["y"].astype(F), oracle.layernorm_fw(x, w, b, rows, width, eps), tol, "layernorm y")
    dx, dw, db = oracle.layernorm_bw(x, w, dy, rows, width, eps)
    assert_close(got["dx"].astype(F), dx, tol, "layernorm dx")
    assert_close(got["dw"].astype(F), dw, tol, "layernorm dw")
    assert_close(got["db"].astype(F), db, tol, "layernorm db")


@pytest.mark.parametrize("half", [False, True], ids=["fp32", "fp16"])
def test_gelu_backward_extension(run, oracle, half):
    rng = seeded(5)
    x = np.concatenate([np.linspace(-6, 6, 1001), rng.standard_normal(3000)]).astype(F); dy = rng.standard_normal(x.size).astype(F)
    if half:
        x, dy = x.astype(np.float16).astype(F), dy.astype(np.float16).astype(F)
    got = run(device=True, half=half).gelu_bw(x, dy)
    assert_close(got.astype(F), oracle.act_bw(3, x, oracle.act_fw(3, x), dy), FP16_TOL if half else FP32_TOL, "gelu dx")


def test_mobilebert_block_fp16_against_its_fp32_twin(pkg, gpulib):
    """config 4: the block of bench_layers.MobileBertBlock (forward, full backward, MSE) in fp16 against the same call
    sequence through the fp32 entry points on the same fp16-representable parameters and inputs.  Every primitive of the
    sequence has its own oracle test above; this one checks the composition and the fp16 error budget (1e-2)."""
    import bench_layers
    runs = {}
    for half in (False, True):
        blk = bench_layers.MobileBertBlock(pkg, gpulib, half=half)
        blk.setup_device()
        blk.step_device()
        gpulib.trainlib_synchronize(); pkg.check(gpulib)
        runs[half] = dict(loss=blk.get("loss"), Y=blk.get("Y"), dX=blk.get("X", grad=True), dWbi=blk.get("Wbi", grad=True), dW1=blk.get("W1_0", grad=True),
                          dW2=blk.get("W2_3", grad=True), dWq=blk.get("Wq", grad=True), dWo=blk.get("Wo", grad=True), dln=blk.get("ln2_w", grad=True), x2=blk.get("x2"))
    assert gpulib.trainlib_tc_status() == 0
    for k in runs[False]:
        assert np.abs(runs[False][k]).max() > 0, "%s is all zero: the call sequence did not reach it" % k
        assert_close(runs[True][k], runs[False][k], FP16_TOL, "block %s (fp16 vs fp32)" % k)
    # the fp32 twin's forward against numpy for the parts that need no reference approximations: first bottleneck + layer norm
    blk = bench_layers.MobileBertBlock(pkg, gpulib, half=False); blk.setup_device(); blk.step_device(); gpulib.trainlib_synchronize()
    X, Wbi, w, b = blk.get("X"), blk.get("Wbi"), blk.get("ln1_w"), blk.get("ln1_b")
    t0 = X.astype(np.float64) @ Wbi.astype(np.float64)
    m = t0.mean(1, keepdims=True); v = ((t0 - m) ** 2).mean(1, keepdims=True)
    assert_close(blk.get("x1"), ((t0 - m) / np.sqrt(v + 1e-3) * w + b).astype(F), 1e-4, "bottleneck + layer norm vs numpy")


def test_mobilebert_block_against_the_cpu_composition(pkg, gpulib, oracle):
    """config 4's block through the fp32 entry points against the same block composed on the CPU from the oracle's
    primitives (tests/block_oracle.py): forward activations, loss, and the gradient of every kind of parameter"""
    import bench_layers
    import block_oracle
    blk = bench_layers.MobileBertBlock(pkg, gpulib, half=False)
    blk.setup_device(); blk.step_device()
    gpulib.trainlib_synchronize(); pkg.check(gpulib)
    P = {n: blk.get(n) for n in blk.params}
    acts, grads = block_oracle.run_block(oracle, P, blk.get("X"), blk.get("target"), blk.HEADS, blk.NFFN, blk.LOSS_SCALE)
    for name, key in (("x1", "x1"), ("att", "att"), ("x2", "x2"), ("Y", "Y"), ("loss", "loss")):
        assert_close(blk.get(name), acts[key].reshape(blk.get(name).shape), 2e-5, "block forward %s" % name)
    for name in ("Wbo", "W2_3", "W1_0", "ln2_w", "ln2_b", "Wq", "Wk", "Wv", "Wo", "ln1_w", "Wbi", "X", "lnf_2_w"):
        assert_close(blk.get(name, grad=True), grads[name].reshape(blk.get(name, grad=True).shape), 5e-5, "block gradient of %s" % name)


@pytest.mark.parametrize("half", [False, True], ids=["fp32", "fp16"])
@pytest.mark.parametrize("sa,sb", [((3, 5, 7), (3, 7, 4)), ((2, 1, 6, 5), (3, 5, 8)), ((1, 4, 9), (2, 3, 1, 9, 2)), ((4, 64, 96), (1, 96, 80)), ((70, 33), (33, 9))])
def test_mm_broadcast(run, oracle, sa, sb, half):
    """NumPy-style batched product (leading dimensions broadcast) against the oracle"""
    rng = seeded(sum(sa) * 3 + sum(sb))
    A = rng.standard_normal(sa).astype(F); B = rng.standard_normal(sb).astype(F)
    if half:
        A, B = A.astype(np.float16).astype(F), B.astype(np.float16).astype(F)
    got = run(device=True, half=half).mm_broadcast(A, B)
    assert_close(got.astype(F), oracle.mm_broadcast(A, B), FP16_TOL if half else FP32_TOL, "mm_broadcast")


@pytest.mark.parametrize("g", [geom(5, 9, 8, 6, 3, pad=0), geom(16, 32, 32, 32, 3, pad=1), geom(8, 16, 16, 12, 3, stride=2, pad=1)],
                         ids=lambda v: "c%d_%dx%d_o%d_s%d_p%d" % (v["Cin"], v["Hin"], v["Win"], v["Cout"], v["sh"], v["padU"]))
def test_conv2d_hwc_layout(run, oracle, g):
    """HWC = 1: activations [H][W][C], weights [Cout][Hk][Wk][Cin]; the same convolution as the CHW oracle on permuted operands"""
    rng = seeded(g["Cin"] * 5 + g["Cout"])
    Ho, Wo = out_hw(g)
    x = rng.uniform(-1, 1, (g["Cin"], g["Hin"], g["Win"])).astype(F); w = rng.uniform(-1, 1, (g["Cout"], g["Cin"], g["Hk"], g["Wk"])).astype(F)
    dy = rng.standard_normal((g["Cout"], Ho, Wo)).astype(F)
    hwc = lambda a: np.ascontiguousarray(a.transpose(1, 2, 0))
    got = run(device=True).conv2d(hwc(x), np.ascontiguousarray(w.transpose(0, 2, 3, 1)), hwc(dy), g, use_im2col=1, hwc=1)
    assert_close(got["y"].reshape(Ho, Wo, g["Cout"]).transpose(2, 0, 1), oracle.conv2d_fw(x, w, None, g), FP32_TOL, "hwc fw")
    assert_close(got["dw"].reshape(g["Cout"], g["Hk"], g["Wk"], g["Cin"]).transpose(0, 3, 1, 2), oracle.conv2d_wg(x, dy, g)[0], FP32_TOL, "hwc wg")
    assert_close(got["dx"].reshape(g["Hin"], g["Win"], g["Cin"]).transpose(2, 0, 1), oracle.conv2d_ig(dy, w, g), FP32_TOL, "hwc ig")


@pytest.mark.gpu
@pytest.mark.parametrize("C,H,W,n", [(16, 32, 32, 3), (32, 16, 16, 2), (64, 8, 8, 5), (6, 12, 12, 2), (3, 7, 7, 1), (4, 40, 40, 1)],
                         ids=["32x32_pair", "16x16_warp", "8x8_half", "12x12_warp1", "7x7_generic", "40x40_generic"])
@pytest.mark.parametrize("with_skip", [False, True], ids=["relu", "skip_relu"])
def test_instnorm_fused_with_sum_and_relu(pkg, gpulib, oracle, C, H, W, n, with_skip):
    """trainlib_instnorm_act_*: one pass must give the bits of norm -> (+ skip) -> ReLU made of the reference's three calls, and
    its backward those of ReLU backward -> norm backward; the three calls themselves are checked against the oracle."""
    rng = seeded(77)
    x = rng.standard_normal((n, C, H, W)).astype(F); gb = rng.standard_normal(2 * C).astype(F); dy = rng.standard_normal(x.shape).astype(F)
    skip = rng.standard_normal(x.shape).astype(F) if with_skip else None
    gpulib.trainlib_set_streams(n)
    try:
        r = AbiRunner(pkg, gpulib, device=True)
        dy2 = rng.standard_normal(x.shape).astype(F) if (C * H * W) % 2 == 0 else None     # a second reader's gradient on some shapes
        fused = r.instnorm_act(x, gb, dy, skip=skip, relu=True, backward=not with_skip, n=n, diff2=None if with_skip else dy2)
        # the separate calls
        X, dX, Y, dY, GB, dGB = r.t(x), r.zeros(*x.shape), r.zeros(*x.shape), r.t(dy), r.t(gb), r.zeros(2 * C)
        m, v, sd = r.zeros(n * C), r.zeros(n * C), r.zeros(n * C)
        a = r.args("InstNorm_args", input=r.blob(X, dX, C=C, H=H, W=W), output=r.blob(Y, dY, C=C, H=H, W=W), coeff=r.blob(GB, dGB, dim=2 * C, W=2 * C),
                   running_mean=m, running_var=v, running_stdev=sd, freeze_running_params=0, skip_wg_grad=0, skip_in_grad=0)
        r.call("pulp_instnorm_fp32_fw_cl", a)
        y_norm = Y.get().copy()
        want = y_norm + skip if with_skip else y_norm          # one fp32 addition per element, as pulp_residualconn_fp32_fw
        want = np.where(want > 0, want, F(0)).astype(F)
        assert np.array_equal(fused["y"], want), "fused forward differs from the three calls"
        assert np.array_equal(fused["mean"], m.get()) and np.array_equal(fused["std"], sd.get())
        for s in range(n):
            o = oracle.instnorm(x[s], gb, dy[s])
            ws = o["y"] + skip[s] if with_skip else o["y"]
            assert_close(fused["y"][s], np.maximum(ws, 0), FP32_TOL, "fused forward vs oracle")
        if not with_skip:
            both = dy + dy2 if dy2 is not None else dy          # pulp_sumnode_fp32_bw
            dY.set(np.where(want > 0, both, F(0)).astype(F))    # pulp_relu_fp32_bw_cl
            r.call("pulp_instnorm_fp32_bw_cl", a)
            assert np.array_equal(fused["dx"], dX.get()), "fused backward dX differs from ReLU backward + norm backward"
            assert np.array_equal(fused["dgb"], dGB.get()), "fused backward parameter gradient differs"
        r.close()
    finally:
        gpulib.trainlib_set_streams(1)


@pytest.mark.gpu
def test_instnorm_fused_fp16_and_rejections(pkg, gpulib):
    """fp16 twin (composed from the separate kernels) and the argument checks of the backward call"""
    rng = seeded(78)
    C, H, W = 8, 16, 16
    x = rng.standard_normal((C, H, W)).astype(np.float16); gb = rng.standard_normal(2 * C).astype(np.float16); dy = rng.standard_normal(x.shape).astype(np.float16)
    r = AbiRunner(pkg, gpulib, device=True, half=True)
    fused = r.instnorm_act(x, gb, dy, relu=True)
    plain = r.instnorm(x, gb, dy)
    want = np.where(plain["y"] > 0, plain["y"], np.float16(0))
    assert np.array_equal(fused["y"], want)
    masked = r.instnorm(x, gb, np.where(want > 0, dy, np.float16(0)).astype(np.float16))
    assert np.array_equal(fused["dx"], masked["dx"]) and np.array_equal(fused["dgb"], masked["dgb"])
    r.close()
    r = AbiRunner(pkg, gpulib, device=True)
    x32 = x.astype(F)
    with pytest.raises(Exception):
        r.instnorm_act(x32, gb.astype(F), dy.astype(F), skip=x32, relu=True, backward=True)    # backward with a skip is refused
    r.close()


@pytest.mark.gpu
@pytest.mark.parametrize("g,n", [(geom(16, 32, 32, 32, 1, stride=2, pad=0), 3), (geom(32, 16, 16, 64, 1, stride=2, pad=0), 2), (geom(6, 9, 9, 4, 1, stride=2, pad=0), 2),
                                 (geom(8, 12, 12, 8, 3, stride=1, pad=1), 2), (geom(4, 8, 8, 6, 1, stride=1, pad=0), 1)],
                         ids=["1x1_s2_16to32", "1x1_s2_32to64", "1x1_s2_odd", "3x3_s1", "1x1_s1"])
def test_conv2d_input_gradient_accumulate(pkg, gpulib, oracle, g, n):
    """trainlib_conv2d_fp32_bw_input_grads_acc_cl: input.diff += dX, against the plain call into a second buffer plus one fp32 sum"""
    rng = seeded(91)
    Ho, Wo = out_hw(g)
    w = rng.uniform(-1, 1, (g["Cout"], g["Cin"], g["Hk"], g["Wk"])).astype(F)
    dy = rng.standard_normal((n, g["Cout"], Ho, Wo)).astype(F); base = rng.standard_normal((n, g["Cin"], g["Hin"], g["Win"])).astype(F)
    gpulib.trainlib_set_streams(n)
    try:
        r = AbiRunner(pkg, gpulib, device=True)
        X, W_, dY, Y = r.zeros(*base.shape), r.t(w), r.t(dy), r.zeros(*dy.shape)
        dX_plain, dX_acc, one = r.zeros(*base.shape), r.t(base), r.zeros(1)
        def args(dx):
            return r.args("Conv2D_args", input=r.blob(X, dx, C=g["Cin"], H=g["Hin"], W=g["Win"]), coeff=r.blob(W_, None, C=g["Cin"], H=g["Hk"], W=g["Wk"], dim=w.size),
                          bias=r.blob(one, one), output=r.blob(Y, dY, C=g["Cout"], H=Ho, W=Wo), Lpad=g["padL"], Rpad=g["padR"], Upad=g["padU"], Dpad=g["padD"],
                          stride_h=g["sh"], stride_w=g["sw"], i2c_buffer=one, bt_buffer=one, USE_BIASES=0, USE_IM2COL=0, HWC=0)
        r.call("pulp_conv2d_fp32_bw_input_grads_cl", args(dX_plain))
        r.call("trainlib_conv2d_fp32_bw_input_grads_acc_cl", args(dX_acc))
        plain, acc = dX_plain.get(), dX_acc.get()
        for s in range(n):
            assert_close(plain[s], oracle.conv2d_ig(dy[s], w, g), FP32_TOL, "plain input gradient")
        assert_close(acc, plain + base, FP32_TOL, "accumulated input gradient")     # the two calls may run on different kernels
        r.close()
    finally:
        gpulib.trainlib_set_streams(1)
