"""GPU parity of the exported entry points that the layer-level tests do not reach: tensor helpers
(layout change, copy, fill, vector sum, casts), the bias-add and mm_manager paths, the naive
convolution kernels called by name, the softmax pieces, mean/std, pointwise convolutions with
C_in != C_out and in HWC, depthwise forward with stride and padding, and the fp16 twins of
pointwise / depthwise conv, CrossEntropy, residual, average pooling, im2row and transpose.

Expected values: the semantics written out in numpy from the reference source cited per test, the
CPU oracle where it has the function, and - when oracle/_ref/libpulp_ref.so travelled with the
repository - the reference's own code driven through the same structs.
Bars: bit-exact for data movement, 1e-5 (fp32) / 1e-2 (fp16 storage) for arithmetic."""
import ctypes
import os

import numpy as np
import pytest

from abi_runner import AbiRunner
from metrics import FP16_TOL, FP32_TOL, assert_close, assert_exact, seeded
from oracle_bind import geom, out_hw

pytestmark = pytest.mark.gpu
F = np.float32
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


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


@pytest.fixture(scope="module")
def ref_runner(pkg):
    """The reference's own C code on the host, or None when the library did not travel."""
    path = os.path.join(ROOT, "oracle", "_ref", "libpulp_ref.so")
    if not os.path.exists(path):
        return None
    return AbiRunner(pkg, pkg.bind(ctypes.CDLL(path)), is_ref=True)


def h16(a):
    return np.asarray(a, F).astype(np.float16).astype(F)


# ------------------------------------------------------------------ data movement (bit-exact)
@pytest.mark.parametrize("device", [False, True])
def test_layout_change_is_bit_exact(run, ref_runner, device):
    """HWC_to_CHW / CHW_to_HWC [ref: lib/sources/pulp_train_utils_fp32.c:821-927]: data and/or gradient of a blob,
    in place, through the caller's transpose buffer"""
    rng = seeded(31)
    C, H, W = 5, 6, 7
    chw = rng.standard_normal((C, H, W)).astype(F); gchw = rng.standard_normal((C, H, W)).astype(F)
    hwc = np.ascontiguousarray(chw.transpose(1, 2, 0)); ghwc = np.ascontiguousarray(gchw.transpose(1, 2, 0))

    def go(r, fn, data, diff, td, tg):
        D, G, buf = r.t(data), r.t(diff), r.zeros(C * H * W)
        args = r.args("layout_args", tensor=r.blob(D, G, C=C, H=H, W=W), transp_buffer=buf, transpose_data=td, transpose_grad=tg)
        r.call(fn, args)
        return D.get().copy().ravel(), G.get().copy().ravel()
    for r in [run(device=device)] + ([ref_runner] if ref_runner else []):
        d, g_ = go(r, "HWC_to_CHW", hwc, ghwc, 1, 1)
        assert_exact(d, chw.ravel(), "HWC_to_CHW data"); assert_exact(g_, gchw.ravel(), "HWC_to_CHW grad")
        d, g_ = go(r, "CHW_to_HWC", chw, gchw, 1, 0)
        assert_exact(d, hwc.ravel(), "CHW_to_HWC data"); assert_exact(g_, gchw.ravel(), "CHW_to_HWC leaves the gradient alone")


@pytest.mark.parametrize("half", [False, True])
def test_copy_fill_sum_are_bit_exact(run, half):
    """copy, set_to_value, vect_sum [ref: lib/sources/pulp_train_utils_fp32.c:186-222] and their fp16 twins"""
    rng = seeded(32)
    n = 1000
    r = run(device=True, half=half)
    dt = r.dt
    a = rng.standard_normal(n).astype(dt); b = rng.standard_normal(n).astype(dt)
    A, B, O = r.t(a), r.t(b), r.zeros(n)
    r.call("copy" + r.sfx, r.args(r.sname("copy_args"), **{"from": A, "to": O, "size": n}))
    assert_exact(O.get(), a, "copy")
    r.call("set_to_value" + r.sfx, r.args(r.sname("set_to_value_args"), to=O, value=0.375, size=n - 3))
    want = a.copy(); want[:n - 3] = dt(0.375)
    assert_exact(O.get(), want, "set_to_value writes `size` elements and no more")
    r.call("vect_sum" + r.sfx, r.args(r.sname("vect_sum_args"), op_1=A, op_2=B, dest=O, size=n))
    assert_exact(O.get(), (a.astype(F) + b.astype(F)).astype(dt), "vect_sum")


def test_casts(run):
    """cast_fp32_tensor_to_fp16 / cast_fp16_tensor_to_fp32 [ref: lib/sources/pulp_train_utils_fp16.c:45-80]: round to nearest even, exact widening"""
    rng = seeded(33)
    n = 777
    x = (rng.standard_normal(n) * 10.0 ** rng.integers(-6, 5, n)).astype(F)
    r = run(device=True)
    X = r.t(x); Hh = Tens16(r, n); Back = r.zeros(n)
    r.call("cast_fp32_tensor_to_fp16", r.args("cast_32t16_args", source=X, destination=Hh.arg, size=n))
    assert_exact(Hh.get(), x.astype(np.float16), "fp32 -> fp16")
    r.call("cast_fp16_tensor_to_fp32", r.args("cast_16t32_args", source=Hh.arg, destination=Back, size=n))
    assert_exact(Back.get(), x.astype(np.float16).astype(F), "fp16 -> fp32")
    Hh.free()


class Tens16(object):
    """a device buffer of n fp16 values beside an fp32 runner"""
    def __init__(self, r, n):
        self.r, self.n = r, n
        self.dev = r.pkg.DeviceBuffer(r.lib, np.zeros(n, np.float16))
        self.arg = self.dev.ptr

    def get(self):
        return self.dev.download(np.float16, (self.n,))

    def free(self):
        self.dev.free()


@pytest.mark.parametrize("half", [False, True])
def test_transpose_and_im2row_fp16_twins(run, oracle, half):
    """transpose (N-d permute) and pulp_im2row: bit-exact in either precision (pure data movement)"""
    rng = seeded(34)
    r = run(device=True, half=half)
    x = rng.standard_normal((3, 4, 5)).astype(r.dt)
    assert_exact(r.transpose(x, (2, 0, 1)), np.ascontiguousarray(x.transpose(2, 0, 1)), "transpose")
    g = geom(3, 7, 6, 4, 3, stride=1, pad=1)
    xi = rng.standard_normal((3, 7, 6)).astype(r.dt)
    Ho, Wo = out_hw(g)
    want = oracle.im2row(xi.astype(F), 3, 7, 6, 3, 3, Ho, Wo, 1, 1, 1, 1).astype(r.dt)
    assert_exact(r.im2row(xi, g), want.ravel(), "im2row")


# ------------------------------------------------------------------ bias add, mm_manager, scalar helpers
@pytest.mark.parametrize("t", [0, 1])
@pytest.mark.parametrize("half", [False, True])
def test_mm_bias_add_transposed(run, ref_runner, t, half):
    """[ref: lib/sources/pulp_train_utils_fp32.c:1286-1323] t = 0: mat[i][j] += bias[j];  t = 1: mat[i][j] += bias[i]"""
    rng = seeded(35 + t)
    H, W = 9, 13
    mat = rng.standard_normal((H, W)).astype(F); bias = rng.standard_normal(H if t else W).astype(F)
    if half:
        mat, bias = h16(mat), h16(bias)
    want = mat + (bias[:, None] if t else bias[None, :])
    runners = [run(device=True, half=half)] + ([ref_runner] if (ref_runner and not half) else [])
    for r in runners:
        M, B = r.t(mat), r.t(bias)
        r.call("mm_bias_add_transposed" + r.sfx, r.args(r.sname("mm_bias_add_args"), mat=M, bias=B, H=H, W=W, t=t))
        assert_close(M.get().astype(F), want, FP16_TOL if half else 1e-7, "mm_bias_add_transposed t=%d" % t)


@pytest.mark.parametrize("bias_transposed", [0, 1])
@pytest.mark.parametrize("trans_B", [0, 1])
def test_mm_manager_product_and_bias(run, oracle, bias_transposed, trans_B):
    """mm_manager [ref: lib/sources/pulp_train_utils_fp32.c:1330-1683]: the selected product, then, with USE_BIASES = 1,
    mm_bias_add_transposed over C[N x M] with t = bias_transposed"""
    rng = seeded(37 + 2 * bias_transposed + trans_B)
    N, K, M = 11, 29, 17
    A = rng.standard_normal((N, K)).astype(F); B = rng.standard_normal((M, K) if trans_B else (K, M)).astype(F)
    bias = rng.standard_normal(N if bias_transposed else M).astype(F)
    want = oracle.mm(A, B, N, K, M, trans_B) + (bias[:, None] if bias_transposed else bias[None, :])
    r = run(device=True)
    a, b, c, bb = r.t(A), r.t(B), r.zeros(N, M), r.t(bias)
    mm_args = r.args("matMul_args", A=a, B=b, C=c, N=N, K=K, M=M, trans_B=trans_B, bias=bb, bias_dim=bias.size, USE_BIASES=1, bias_transposed=bias_transposed)
    for layer, step in ((3, 0), (0, 0), (2, 2)):     # LAYER_LINEAR forward, LAYER_CONV2D forward, LAYER_PW_CONV input gradient
        r.call("mm_manager", r.args("mm_manager_args", mm_args=mm_args, layer_type=layer, step_type=step, matmul_type=10))
        assert_close(c.get(), want, FP32_TOL, "mm_manager layer %d" % layer)
    # without the flag the bias pointer is ignored
    mm_args.USE_BIASES = 0
    r.call("mm_manager", r.args("mm_manager_args", mm_args=mm_args, layer_type=3, step_type=0, matmul_type=0))
    assert_close(c.get(), oracle.mm(A, B, N, K, M, trans_B), FP32_TOL, "mm_manager without bias")


def test_scalar_mul_row_pieces_mean_std(run, ref_runner, oracle):
    """pulp_scalar_mul_fp32_cl [ref: pulp_train_utils_fp32.c:1191]; the softmax pieces pulp_row_max / pulp_exp_sum / pulp_row_div
    [ref: :1046-1189] (exp = the reference's bit-trick fastexp_gist); pulp_mean_std_fp32_cl [ref: :1693-1730]"""
    rng = seeded(39)
    H, W = 12, 37
    x = rng.standard_normal((H, W)).astype(F)

    def pieces(r):
        X, mx, out, sums = r.t(x), r.t(np.full(H, -np.inf, F) if not r.is_ref else np.full(H, -3.0e38, F)), r.zeros(H, W), r.zeros(H)
        r.call("pulp_row_max_fp32_cl", r.args("max_args", input=X, H=H, W=W, maxes=mx))
        r.call("pulp_exp_sum_fp32_cl", r.args("exp_sum_args", input=X, output=out, H=H, W=W, maxes=mx, sums=sums))
        e = out.get().copy()
        r.call("pulp_row_div_fp32_cl", r.args("row_div_args", input=out, H=H, W=W, sums=sums))
        sc = r.t(x.ravel())
        r.call("pulp_scalar_mul_fp32_cl", r.args("scalar_mul_args", input=sc, scalar=0.3125, dim=H * W))
        m, v, s = r.zeros(1), r.zeros(1), r.zeros(1)
        r.call("pulp_mean_std_fp32_cl", r.args("mean_std_args", input=X, mean=m, var=v, std=s, epsilon=1e-5, dim=H * W))
        return dict(max=mx.get().copy(), exp=e, sums=sums.get().copy(), soft=out.get().copy(), scaled=sc.get().copy(),
                    mean=m.get().copy(), var=v.get().copy(), std=s.get().copy())
    got = pieces(run(device=True))
    assert_exact(got["max"], x.max(axis=1), "row max")
    assert_exact(got["scaled"], (x.ravel() * F(0.3125)), "scalar mul")
    assert_close(got["soft"], oracle.softmax_fw(x), FP32_TOL, "row_max + exp_sum + row_div = softmax forward")
    assert_close(got["sums"], got["exp"].sum(axis=1), FP32_TOL, "row sums of the exponentials")
    xm = x.astype(np.float64)
    assert_close(got["mean"], [xm.mean()], FP32_TOL, "mean"); assert_close(got["var"], [xm.var() + 1e-5], 2e-5, "var + eps")
    assert_close(got["std"], [np.sqrt(xm.var() + 1e-5)], FP32_TOL, "std")
    if ref_runner:
        want = pieces(ref_runner)
        for k in ("max", "scaled"):
            assert_exact(got[k], want[k], k + " vs reference")
        for k in ("exp", "sums", "soft", "mean", "var", "std"):
            assert_close(got[k], want[k], FP32_TOL, k + " vs reference")


# ------------------------------------------------------------------ convolutions by other doors
def test_naive_conv_kernels_by_name(run, oracle):
    """naive_conv2d_{fw,param_grad,in_grad}_kernel_CHW [ref: lib/sources/pulp_conv_naive_fp32.c:198-516] take a matMul_args with
    A = input (or its gradient), B = weights (or their gradient), C = output (or its gradient) and the geometry fields"""
    rng = seeded(40)
    g = geom(5, 9, 8, 7, 3, stride=2, pad=1)
    Ho, Wo = out_hw(g)
    x = rng.uniform(-1, 1, (5, 9, 8)).astype(F); w = rng.uniform(-1, 1, (7, 5, 3, 3)).astype(F); dy = rng.standard_normal((7, Ho, Wo)).astype(F)
    bias = rng.standard_normal(7).astype(F)
    r = run(device=True)
    geo = dict(H=g["Hin"], W=g["Win"], pH=3, pW=3, pCin=5, pCout=7, stride_h=2, stride_w=2, Lpad=1, Rpad=1, Upad=1, Dpad=1, HWC=0)
    X, W_, Y, Bt = r.t(x), r.t(w), r.zeros(7, Ho, Wo), r.t(bias)
    r.call("naive_conv2d_fw_kernel_CHW", r.args("matMul_args", A=X, B=W_, C=Y, bias=Bt, USE_BIASES=1, **geo))
    assert_close(Y.get(), oracle.conv2d_fw(x, w, bias, g), FP32_TOL, "naive fw")
    dW, dY, dB = r.zeros(*w.shape), r.t(dy), r.zeros(7)
    r.call("naive_conv2d_param_grad_kernel_CHW", r.args("matMul_args", A=X, B=dW, C=dY, bias=dB, USE_BIASES=1, **geo))
    want_dw, want_db = oracle.conv2d_wg(x, dy, g, with_bias=True)
    assert_close(dW.get(), want_dw, FP32_TOL, "naive wg"); assert_close(dB.get(), want_db, FP32_TOL, "naive bias grad")
    dX = r.zeros(*x.shape)
    r.call("naive_conv2d_in_grad_kernel_CHW", r.args("matMul_args", A=dX, B=W_, C=dY, USE_BIASES=0, **geo))
    assert_close(dX.get(), oracle.conv2d_ig(dy, w, g), FP32_TOL, "naive ig")


@pytest.mark.parametrize("half", [False, True])
@pytest.mark.parametrize("Cin,Cout,hwc", [(8, 8, 0), (6, 20, 0), (24, 5, 0), (6, 20, 1), (8, 8, 1)])
def test_pointwise_conv(run, oracle, Cin, Cout, hwc, half):
    """pulp_conv_pw_* [ref: lib/sources/pulp_conv_pw_fp32.c:27-330] against the 1x1 convolution of the oracle, also where
    C_in != C_out (the reference's own input gradient swaps two dimensions there) and in HWC"""
    rng = seeded(41 + Cin + Cout)
    H, W = 6, 5
    g = geom(Cin, H, W, Cout, 1)
    x = rng.uniform(-1, 1, (Cin, H, W)).astype(F); w = rng.uniform(-1, 1, (Cout, Cin, 1, 1)).astype(F); dy = rng.standard_normal((Cout, H, W)).astype(F)
    if half:
        x, w, dy = h16(x), h16(w), h16(dy)
    want = dict(y=oracle.conv2d_fw(x, w, None, g), dw=oracle.conv2d_wg(x, dy, g)[0], dx=oracle.conv2d_ig(dy, w, g))
    r = run(device=True, half=half)
    if hwc:
        xi, dyi = np.ascontiguousarray(x.transpose(1, 2, 0)), np.ascontiguousarray(dy.transpose(1, 2, 0))
        # HWC: activations [H][W][C], coefficients [C_in][C_out] (the reference multiplies X[HW x C_in] by them untransposed, :75-81)
        wi = np.ascontiguousarray(w.reshape(Cout, Cin).T)
        got = r.pw(xi.astype(r.dt), wi.astype(r.dt), dyi.astype(r.dt), Cin, Cout, H, W, hwc=1)
        got = dict(y=got["y"].reshape(H, W, Cout).transpose(2, 0, 1), dw=got["dw"].reshape(Cin, Cout).T, dx=got["dx"].reshape(H, W, Cin).transpose(2, 0, 1))
    else:
        got = r.pw(x.astype(r.dt), w.astype(r.dt), dy.astype(r.dt), Cin, Cout, H, W)
    tol = FP16_TOL if half else FP32_TOL
    for k in ("y", "dw", "dx"):
        assert_close(np.asarray(got[k], F).reshape(want[k].shape), want[k], tol, "pointwise %s" % k)


@pytest.mark.parametrize("half", [False, True])
@pytest.mark.parametrize("stride,pad", [(1, 0), (1, 1), (2, 1)])
def test_depthwise_conv(run, oracle, stride, pad, half):
    """pulp_conv_dw_* [ref: lib/sources/pulp_conv_dw_fp32.c:27-86, pulp_conv_naive_fp32.c:29-194]: the forward honours stride
    and padding; the gradients are checked where the reference's are defined (stride 1, no padding) and against the
    correct convolution otherwise"""
    rng = seeded(50 + 3 * stride + pad)
    C, H, W, k = 6, 9, 10, 3
    g = dict(geom(C, H, W, C, k, stride=stride, pad=pad))
    Ho, Wo = out_hw(g)
    x = rng.uniform(-1, 1, (C, H, W)).astype(F); w = rng.uniform(-1, 1, (C, k, k)).astype(F); dy = rng.standard_normal((C, Ho, Wo)).astype(F)
    if half:
        x, w, dy = h16(x), h16(w), h16(dy)
        if stride != 1:
            pytest.skip("DepthWise_Conv_args_fp16 has no stride fields")
    r = run(device=True, half=half)
    got = r.dw(x.astype(r.dt), w.astype(r.dt), dy.astype(r.dt), g)
    tol = FP16_TOL if half else FP32_TOL
    assert_close(got["y"].astype(F), oracle.dw_fw(x, w, g), tol, "depthwise fw s%d p%d" % (stride, pad))
    assert_close(got["dw"].astype(F), oracle.dw_wg(x, dy, g), tol, "depthwise wg")
    assert_close(got["dx"].astype(F), oracle.dw_ig(dy, w, g), tol, "depthwise ig")


def test_fp16_twins_of_loss_residual_pool(run, oracle):
    """fp16 storage twins of CrossEntropy, the residual trio and average pooling against the fp32 oracle on the rounded inputs"""
    rng = seeded(60)
    r = run(device=True, half=True)
    z = h16(rng.standard_normal(10) * 2); t = np.zeros(10, F); t[3] = 1
    loss, dz = r.loss("CrossEntropyLoss", z.astype(np.float16), t.astype(np.float16))
    wl, wdz = oracle.ce(z, t)
    assert_close([loss], [wl], FP16_TOL, "CrossEntropy fp16"); assert_close(dz.astype(F), wdz, FP16_TOL, "CrossEntropy backward fp16")
    a, b, d, e = [h16(rng.standard_normal(200)) for _ in range(4)]
    res = r.residual(a.astype(np.float16), b.astype(np.float16), d.astype(np.float16), e.astype(np.float16))
    assert_close(res["out"].astype(F), a + b, FP16_TOL, "residual fw fp16")
    assert_close(res["dskip"].astype(F), e + d, FP16_TOL, "sumnode bw fp16"); assert_close(res["dlout"].astype(F), d, FP16_TOL, "residual bw fp16")
    x = h16(rng.standard_normal((4, 8, 8))); dyp = h16(rng.standard_normal((4, 4, 4)))
    got = r.avgpool(x.astype(np.float16), dyp.astype(np.float16), 2, 2, 2, 2)
    want = oracle.avgpool(x, dyp, 2, 2, 2, 2)
    assert_close(got["y"].astype(F), want[0], FP16_TOL, "avgpool fw fp16"); assert_close(got["dx"].astype(F), want[1], FP16_TOL, "avgpool bw fp16")


# ------------------------------------------------------------------ names that alias one implementation
FP16_MM_NAMES = ["mm_fp16_SIMD_2x4", "mm_fp16_SIMD_4x8", "mm_fp16_unroll_8x1", "mm_fp16_unroll_4x1", "mm_fp16_unroll_2x1", "mm_M_fp16_SIMD_2x4", "mm_M_fp16_SIMD_4x8"]


@pytest.mark.parametrize("fn", FP16_MM_NAMES + ["mv_fp16_SIMD_2x1", "mv_fp16_SIMD_4x1", "mv_fp16_SIMD_8x1"])
def test_fp16_matmul_variants_by_name(run, oracle, fn):
    """[ref: lib/include/pulp_matmul_fp16.h:56-134] every variant name computes the product of mm_fp16 (the mv_* names with M = 1)"""
    rng = seeded(70)
    N, K, M = 24, 40, (1 if fn.startswith("mv_") else 16)
    A = h16(rng.standard_normal((N, K))); B = h16(rng.standard_normal((K, M)))
    got = run(device=True, half=True).mm(A.astype(np.float16), B.astype(np.float16), N, K, M, fn=fn)
    assert_close(got.astype(F), oracle.mm(A, B, N, K, M), FP16_TOL, fn)


@pytest.mark.parametrize("half", [False, True])
def test_fixed_geometry_naive_kernels_and_workers(run, oracle, half):
    """naive_conv2d_*_k3x3_s2_p1 ignore the struct's kernel size, stride and padding [ref: lib/sources/pulp_conv_naive_fp32.c:520-700];
    the forked Linear / im2col-convolution workers take a mm_manager_args [ref: lib/sources/pulp_linear_fp32.c:199-267,
    pulp_conv2d_fp32.c:669-742]; HWC_to_CHW_fp16 is the fp16 layout change"""
    rng = seeded(71)
    g = geom(4, 10, 8, 6, 3, stride=2, pad=1)
    Ho, Wo = out_hw(g)
    cast = h16 if half else (lambda a: np.asarray(a, F))
    x = cast(rng.uniform(-1, 1, (4, 10, 8))); w = cast(rng.uniform(-1, 1, (6, 4, 3, 3))); dy = cast(rng.standard_normal((6, Ho, Wo)))
    r = run(device=True, half=half)
    tol = FP16_TOL if half else FP32_TOL
    wrong = dict(H=10, W=8, pH=7, pW=7, pCin=4, pCout=6, stride_h=1, stride_w=1, Lpad=0, Rpad=0, Upad=0, Dpad=0, HWC=0)   # geometry fields the fixed forms must ignore
    X, W_, Y, dW, dX, dY = r.t(x), r.t(w), r.zeros(6, Ho, Wo), r.zeros(*w.shape), r.zeros(*x.shape), r.t(dy)
    sfx = "_fp16" if half else ""
    r.call("naive_conv2d_fw_kernel_CHW_k3x3_s2_p1" + sfx, r.args(r.sname("matMul_args"), A=X, B=W_, C=Y, USE_BIASES=0, **wrong))
    assert_close(Y.get().astype(F), oracle.conv2d_fw(x, w, None, g), tol, "fixed 3x3 s2 p1 fw")
    r.call("naive_conv2d_param_grad_kernel_CHW_k3x3_s2_p1" + sfx, r.args(r.sname("matMul_args"), A=X, B=dW, C=dY, USE_BIASES=0, **wrong))
    assert_close(dW.get().astype(F), oracle.conv2d_wg(x, dy, g)[0], tol, "fixed 3x3 s2 p1 wg")
    r.call("naive_conv2d_in_grad_kernel_CHW_k3x3_s2_p1" + sfx, r.args(r.sname("matMul_args"), A=dX, B=W_, C=dY, USE_BIASES=0, **wrong))
    assert_close(dX.get().astype(F), oracle.conv2d_ig(dy, w, g), tol, "fixed 3x3 s2 p1 ig")
    # forked workers on a mm_manager_args
    N, K, M = 9, 21, 13
    A = cast(rng.standard_normal((N, K))); B = cast(rng.standard_normal((K, M))); bias = cast(rng.standard_normal(N))
    a, b, c, bb = r.t(A), r.t(B), r.zeros(N, M), r.t(bias)
    mm_args = r.args(r.sname("matMul_args"), A=a, B=b, C=c, N=N, K=K, M=M, trans_B=0, bias=bb, USE_BIASES=1, HWC=0)
    man = r.args(r.sname("mm_manager_args"), mm_args=mm_args, layer_type=0, step_type=0, matmul_type=0)
    prod = oracle.mm(A, B, N, K, M)
    r.call("im2col_conv2d_fw_kernel" + sfx, man)
    assert_close(c.get().astype(F), prod + bias[:, None], tol, "im2col_conv2d_fw_kernel: product + bias per output channel")
    r.call(r.fname("pulp_linear_fp32_fw_cl_kernel"), man)
    assert_close(c.get().astype(F), prod, tol, "pulp_linear_fw_cl_kernel: the product, no bias step")
    r.call(r.fname("pulp_linear_fp32_bw_param_grads_cl_kernel"), man)
    assert_close(c.get().astype(F), prod, tol, "pulp_linear_bw_param_grads_cl_kernel product")
    assert_exact(bb.get().astype(F), A.ravel()[:N], "bias gradient = first N values of A")
    if half:
        C_, H, W = 3, 4, 5
        chw = rng.standard_normal((C_, H, W)).astype(np.float16); hwc = np.ascontiguousarray(chw.transpose(1, 2, 0))
        D, G, buf = r.t(hwc), r.zeros(C_ * H * W), r.zeros(C_ * H * W)
        r.call("HWC_to_CHW_fp16", r.args("layout_args_fp16", tensor=r.blob(D, G, C=C_, H=H, W=W), transp_buffer=buf, transpose_data=1, transpose_grad=0))
        assert_exact(D.get().ravel(), chw.ravel(), "HWC_to_CHW_fp16")
        r.call("CHW_to_HWC_fp16", r.args("layout_args_fp16", tensor=r.blob(D, G, C=C_, H=H, W=W), transp_buffer=buf, transpose_data=1, transpose_grad=0))
        assert_exact(D.get().ravel(), hwc.ravel(), "CHW_to_HWC_fp16")


def test_cluster_bringup_runs_a_task_on_the_gpu(pkg):
    """the main.c-style bring-up of tests/test_abi_cpu.py on a box that has a device: pi_cluster_open succeeds, the task's
    padded convolution runs through the host-pointer path and its checksum matches numpy"""
    import test_abi_cpu
    test_abi_cpu.test_cluster_bringup_links_and_runs(pkg)


def test_elementwise_family_fp16(pkg, gpulib):
    """fp16 twins of L1 / berHu, max pooling, NoNorm, RMS norm, SwiGLU, vector softmax and the softmax pieces against the
    float32 restatement on fp16-representable inputs; host-pointer and device-pointer calls give the same bits"""
    import golden_cases
    name, make_inputs, _, _, _ = [c for c in golden_cases.CASES if c[0] == "elementwise_family"][0]
    i = make_inputs(np.random.default_rng(golden_cases.case_seed(name)))
    i = {k: v.astype(np.float16).astype(np.float32) for k, v in i.items()}
    want = golden_cases.family_oracle(i, with_shift=False)
    r = AbiRunner(pkg, gpulib, device=True, half=True)
    got = r.family(i)
    r.close()
    for k, w in want.items():
        tol = 3e-2 if k in ("berhu", "berhu_dy", "mp3_dx", "rmsnorm") else 1e-2      # a rounded threshold c / sums of rounded terms
        assert_close(got[k].astype(np.float32), w, tol, "fp16 family %s" % k)
    rh = AbiRunner(pkg, gpulib, device=False, half=True)
    host = rh.family(i)
    rh.close()
    for k in want:
        assert_exact(host[k], got[k], "fp16 family %s: host pointers vs device pointers" % k)


def test_maxpool_rejects_a_wrong_output_size(pkg, gpulib):
    r = AbiRunner(pkg, gpulib, device=True)
    X, dX, O, dO = r.zeros(2, 8, 8), r.zeros(2, 8, 8), r.zeros(2, 3, 3), r.zeros(2, 3, 3)
    pa = r.args("pool_args", input=r.blob(X, dX, C=2, H=8, W=8), output=r.blob(O, dO, C=2, H=3, W=3), Hker=2, Wker=2, Hstride=2, Wstride=2)
    import ctypes
    gpulib.pulp_maxpool_fp32_fw_cl(ctypes.byref(pa))
    assert gpulib.trainlib_last_error() == 3          # TL_ERR_BAD_ARGS
    gpulib.trainlib_clear_error()
    r.close()


@pytest.mark.parametrize("half", [False, True])
def test_depthwise_workers_by_name(pkg, gpulib, oracle, half):
    """dw_kernel_forward / weight_grad / input_grad (kernel_DW_args): the fp32 struct carries stride and padding, the fp16 one
    only the blobs (stride 1, no padding)"""
    rng = seeded(41)
    C, H, W, k = 5, 11, 9, 3
    sh, pad = (1, 0) if half else (2, 1)
    g = dict(geom(C, H, W, C, k, stride=sh, pad=pad))
    Ho, Wo = out_hw(g)
    cast = (lambda a: a.astype(np.float16).astype(np.float32)) if half else (lambda a: a)
    x, w, dy = cast(rng.standard_normal((C, H, W)).astype(np.float32)), cast(rng.standard_normal((C, k, k)).astype(np.float32)), cast(rng.standard_normal((C, Ho, Wo)).astype(np.float32))
    r = AbiRunner(pkg, gpulib, device=True, half=half)
    X, dX, Wt, dW, Y, dY = r.t(x), r.zeros(C, H, W), r.t(w), r.zeros(C, k, k), r.zeros(C, Ho, Wo), r.t(dy)
    blobs = dict(input=r.blob(X, dX, C=C, H=H, W=W), weights=r.blob(Wt, dW, C=C, H=k, W=k, dim=w.size), output=r.blob(Y, dY, C=C, H=Ho, W=Wo))
    if half:
        args = r.args("kernel_DW_args_fp16", **blobs)
    else:
        args = r.args("kernel_DW_args", stride_h=sh, stride_w=sh, Lpad=pad, Rpad=pad, Upad=pad, Dpad=pad, **blobs)
    sfx = "_fp16" if half else ""
    for fn in ("dw_kernel_forward", "dw_kernel_weight_grad", "dw_kernel_input_grad"):
        r.call(fn + sfx, args)
    tol = FP16_TOL if half else FP32_TOL
    assert_close(Y.get().astype(np.float32), oracle.dw_fw(x, w, g), tol, "dw_kernel_forward")
    assert_close(dW.get().astype(np.float32), oracle.dw_wg(x, dy, g), tol, "dw_kernel_weight_grad")
    assert_close(dX.get().astype(np.float32), oracle.dw_ig(dy, w, g), tol, "dw_kernel_input_grad")
    r.close()


def test_profile_credits_useful_flops_to_the_kernel_that_ran(pkg, gpulib):
    """trainlib_profile: every convolution launch is credited 2 x (multiply-adds of the operator's definition); the bench's
    roofline fractions are built on these figures, so they are checked here against the closed form"""
    rng = seeded(77)
    n, C, H = 40, 16, 32
    g = dict(geom(C, H, H, C, 3, pad=1))
    xs = rng.uniform(-1, 1, (n, C, H, H)).astype(np.float32); w = rng.uniform(-1, 1, (C, C, 3, 3)).astype(np.float32)
    gpulib.trainlib_set_streams(n)
    try:
        r = AbiRunner(pkg, gpulib, device=True)
        X, W_, dY = r.t(xs), r.t(w), r.t(xs)
        Y, dX, dW, one = r.zeros(n, C, H, H), r.zeros(n, C, H, H), r.zeros(C, C, 3, 3), r.zeros(1)
        args = r.args("Conv2D_args", input=r.blob(X, dX, C=C, H=H, W=H), coeff=r.blob(W_, dW, C=C, H=3, W=3, dim=w.size), bias=r.blob(one, one),
                      output=r.blob(Y, dY, C=C, H=H, W=H), Lpad=1, Rpad=1, Upad=1, Dpad=1, stride_h=1, stride_w=1, i2c_buffer=one, bt_buffer=one,
                      USE_BIASES=0, USE_IM2COL=1, HWC=0)
        gpulib.trainlib_profile(1)
        for fn in ("pulp_conv2d_fp32_fw_cl", "pulp_conv2d_fp32_bw_input_grads_cl", "pulp_conv2d_fp32_bw_param_grads_cl"):
            r.call(fn, args)
        gpulib.trainlib_profile(0)
        table = pkg.profile_table(gpulib, flops=True)
        want = 2.0 * n * C * C * 9 * H * H
        credited = sum(row[3] for row in table)
        assert abs(credited - 3 * want) <= 1e-6 * want, (credited, 3 * want, table)
        assert all(row[3] == 0.0 for row in table if "reduce" in row[0] or "column" in row[0])
        r.close()
    finally:
        gpulib.trainlib_set_streams(1)


@pytest.mark.gpu
def test_deferred_reductions_give_the_same_bits_in_one_launch(pkg, gpulib):
    """trainlib_set_deferred_reductions: the weight gradients of four convolutions (FFMA, tcgen05 stride 1 and 2, 1x1 strided
    kernels) and the parameter gradient of an instance norm, issued back to back, are summed by one batched launch at
    the flush, with the bits of the immediate mode"""
    cases = [(geom(16, 32, 32, 16, 3, pad=1), 40), (geom(32, 16, 16, 32, 3, pad=1), 300), (geom(16, 32, 32, 32, 1, stride=2), 33),
             (geom(32, 16, 16, 64, 3, stride=2, pad=1), 260)]
    results = {}
    for mode in (0, 1):
        r = AbiRunner(pkg, gpulib, device=True)
        outs, calls = [], []
        for g, n in cases:
            Ho, Wo = out_hw(g)
            rs = np.random.default_rng(g["Cin"] + n)
            xs = rs.uniform(-1, 1, (n, g["Cin"], g["Hin"], g["Win"])).astype(np.float32); dys = rs.standard_normal((n, g["Cout"], Ho, Wo)).astype(np.float32)
            X, dY, dW, one = r.t(xs), r.t(dys), r.zeros(g["Cout"], g["Cin"], g["Hk"], g["Wk"]), r.zeros(1)
            args = r.args("Conv2D_args", input=r.blob(X, one, C=g["Cin"], H=g["Hin"], W=g["Win"]), coeff=r.blob(one, dW, C=g["Cin"], H=g["Hk"], W=g["Wk"], dim=g["Cout"] * g["Cin"] * g["Hk"] * g["Wk"]),
                          bias=r.blob(one, one), output=r.blob(one, dY, C=g["Cout"], H=Ho, W=Wo), Lpad=g["padL"], Rpad=g["padR"], Upad=g["padU"], Dpad=g["padD"],
                          stride_h=g["sh"], stride_w=g["sw"], i2c_buffer=one, bt_buffer=one, USE_BIASES=0, USE_IM2COL=1, HWC=0)
            calls.append((n, "pulp_conv2d_fp32_bw_param_grads_cl", args)); outs.append(dW)
        n, C, H = 200, 16, 32
        rng = seeded(123)
        xs = rng.standard_normal((n, C, H, H)).astype(np.float32); dys = rng.standard_normal((n, C, H, H)).astype(np.float32)
        X, dX, Y, dY, GB, dGB = r.t(xs), r.zeros(n, C, H, H), r.zeros(n, C, H, H), r.t(dys), r.t(np.ones(2 * C, np.float32)), r.zeros(2 * C)
        m, v, s = r.zeros(n * C), r.zeros(n * C), r.zeros(n * C)
        nargs = r.args("InstNorm_args", input=r.blob(X, dX, C=C, H=H, W=H), output=r.blob(Y, dY, C=C, H=H, W=H), coeff=r.blob(GB, dGB, dim=2 * C, W=2 * C),
                       running_mean=m, running_var=v, running_stdev=s, freeze_running_params=0, skip_wg_grad=0, skip_in_grad=0)
        gpulib.trainlib_set_streams(n); r.call("pulp_instnorm_fp32_fw_cl", nargs)
        calls.append((n, "pulp_instnorm_fp32_bw_cl", nargs)); outs.append(dGB)
        gpulib.trainlib_set_deferred_reductions(mode)
        for n_, fn, a in calls:                     # the first pass in the mode sizes the arena of partial results (its sums run at once)
            gpulib.trainlib_set_streams(n_); r.call(fn, a)
        gpulib.trainlib_flush_reductions()
        for o in outs:
            gpulib.trainlib_memset(o.dev.ptr, 0, o.dev.nbytes)
        gpulib.trainlib_profile(1)
        try:
            for n_, fn, a in calls:
                gpulib.trainlib_set_streams(n_); r.call(fn, a)
            gpulib.trainlib_flush_reductions()
        finally:
            gpulib.trainlib_profile(0); gpulib.trainlib_set_deferred_reductions(0); gpulib.trainlib_set_streams(1)
        table = {row[0].strip("()").split("<")[0]: row[1] for row in pkg.profile_table(gpulib)}
        sums = sum(table.get(k, 0) for k in ("reduce_partials_kernel", "reduce_partials_f32_kernel", "wgt_reduce_kernel", "column_direct_kernel", "column_partial_kernel"))
        if mode:
            assert table.get("deferred_reduce_kernel", 0) == 1 and sums == 0, table
        else:
            assert "deferred_reduce_kernel" not in table and sums == 5, table
        results[mode] = [o.get().copy() for o in outs]
        r.close()
    for k, (a, b) in enumerate(zip(results[0], results[1])):
        assert np.abs(a).max() > 0 and np.array_equal(a, b), "deferred and immediate sums differ: output %d, %d of %d elements, max |a| %g, max |a - b| %g" % (
            k, int((a != b).sum()), a.size, float(np.abs(a).max()), float(np.abs(a - b).max()))
