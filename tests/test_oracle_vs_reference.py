"""Pins the CPU restatement (oracle/trainlib_oracle.c) against the reference's own C sources
compiled for the host (oracle/_ref/libpulp_ref.so), function by function, on seeded inputs.
Also validates the ABI harness itself, since the reference is driven through the same structs.
CPU only."""
import numpy as np
import pytest

from abi_runner import AbiRunner
from metrics import assert_close, assert_exact, seeded
from oracle_bind import geom, out_hw

TIGHT = 2e-6      # same formulas in the same order: only libm / contraction noise is allowed


@pytest.fixture()
def ref(pkg, reflib):
    r = AbiRunner(pkg, reflib, is_ref=True)
    yield r
    r.close()


def test_scalar_bit_tricks(oracle, pkg):
    # known answers: q_rsqrt(64) = 0x3dff910f, q_rsqrt(32) ~ 0.17673251 (values of the reference's own golden model, tests/test_mhsa_fp32/utils/mhsa.py)
    assert np.float32(oracle.q_rsqrt(64.0)).view(np.uint32) == 0x3DFF910F
    assert abs(oracle.q_rsqrt(32.0) - 0.17673251) < 1e-7
    assert oracle.fastexp_gist(0.0) == np.float32(np.uint32(1064986823).view(np.float32)) or abs(oracle.fastexp_gist(0.0) - 1.0) < 0.05
    assert oracle.fastexp_gist(-100.0) == 0.0


@pytest.mark.parametrize("N,K,M", [(1, 1, 1), (3, 5, 7), (17, 13, 9), (32, 144, 64), (8, 1, 8), (1, 64, 33)])
@pytest.mark.parametrize("trans_B", [0, 1])
def test_mm(oracle, ref, N, K, M, trans_B):
    rng = seeded(N * 1000 + K * 10 + M + trans_B)
    A = rng.standard_normal((N, K)).astype(np.float32)
    B = rng.standard_normal((M, K) if trans_B else (K, M)).astype(np.float32)
    got = oracle.mm(A, B, N, K, M, trans_B)
    for fn in ("mm", "mm_M", "mm_unroll_2x4", "mm_M_unroll_4x4"):
        assert_exact(got, ref.mm(A, B, N, K, M, trans_B, fn=fn), "mm vs %s" % fn)


@pytest.mark.parametrize("case", [geom(8, 8, 8, 8, 3), geom(3, 9, 7, 5, 3), geom(4, 6, 6, 6, 1), geom(16, 32, 32, 32, 3, pad=1),
                                  geom(6, 10, 10, 4, 3, stride=2, pad=1), geom(5, 9, 9, 7, 5, pad=2)])
def test_conv2d(oracle, ref, case):
    g = case
    rng = seeded(g["Cin"] * 100 + g["Hk"])
    Ho, Wo = out_hw(g)
    x = rng.uniform(-1, 1, (g["Cin"], g["Hin"], g["Win"])).astype(np.float32)
    w = rng.uniform(-1, 1, (g["Cout"], g["Cin"], g["Hk"], g["Wk"])).astype(np.float32)
    dy = rng.standard_normal((g["Cout"], Ho, Wo)).astype(np.float32)
    bias = rng.standard_normal(g["Cout"]).astype(np.float32)
    # naive path of the reference: right for every stride/pad (input grad with pad 0 only for k in {1,3})
    r = ref.conv2d(x, w, dy, g, use_im2col=0, bias=bias)
    assert_close(oracle.conv2d_fw(x, w, bias, g), r["y"], TIGHT, "fw")
    dw, db = oracle.conv2d_wg(x, dy, g, with_bias=True)
    assert_close(dw, r["dw"], TIGHT, "wg")
    if g["padU"] == 0:
        # with padding the reference keeps the bias sum of the LAST tap only, which skips the
        # border pixels that tap cannot reach (lib/sources/pulp_conv_naive_fp32.c:383-398)
        assert_close(db, r["db"], TIGHT, "bias grad")
    else:
        assert_close(db, dy.reshape(g["Cout"], -1).sum(axis=1), 1e-5, "bias grad = plain channel sum")
    if g["padU"] > 0 or g["Hk"] in (1, 3):
        assert_close(oracle.conv2d_ig(dy, w, g), r["dx"], TIGHT, "ig")
    # im2col path of the reference: forward with pad <= 1, everything with pad 0 and stride 1
    if g["sh"] == 1 and g["padU"] <= 1:
        r2 = ref.conv2d(x, w, dy, g, use_im2col=1, steps=("fw",) if g["padU"] else ("fw", "wg", "ig"))
        assert_close(oracle.conv2d_fw(x, w, None, g), r2["y"], TIGHT, "fw im2col")
        if not g["padU"]:
            assert_close(dw, r2["dw"], TIGHT, "wg im2col")
            assert_close(oracle.conv2d_ig(dy, w, g), r2["dx"], TIGHT, "ig im2col")


@pytest.mark.parametrize("pad", [0, 1])
def test_im2row_and_blocktransp(oracle, ref, pad):
    g = geom(4, 7, 6, 5, 3, pad=pad)
    rng = seeded(7 + pad)
    Ho, Wo = out_hw(g)
    x = rng.standard_normal((g["Cin"], g["Hin"], g["Win"])).astype(np.float32)
    dy = rng.standard_normal((g["Cout"], Ho, Wo)).astype(np.float32)
    assert_exact(oracle.im2row(x, g["Cin"], g["Hin"], g["Win"], 3, 3, Ho, Wo, 1, 1, pad, pad), ref.im2row(x, g, mod=0), "im2row fw")
    if pad == 0:
        assert_exact(oracle.im2row(dy, g["Cout"], g["Hin"], g["Win"], 3, 3, Ho, Wo, 1, 1, 0, 0, mode_ig=1), ref.im2row(dy, g, mod=1), "im2row ig")
        assert_exact(oracle.im2row(x, g["Cin"], g["Hin"], g["Win"], 3, 3, Ho, Wo, 1, 1, 0, 0, transposed=1),
                     ref.im2row(x, g, mod=0, fn="pulp_im2col_fp32"), "im2col")
        xh = np.ascontiguousarray(x.transpose(1, 2, 0))
        assert_exact(oracle.im2row(xh, g["Cin"], g["Hin"], g["Win"], 3, 3, Ho, Wo, 1, 1, 0, 0, hwc=1), ref.im2row(xh, g, mod=0, hwc=1), "im2row hwc")
    w = rng.standard_normal((5, 4, 3, 3)).astype(np.float32)
    assert_exact(oracle.blocktransp(w, 4, 5, 3, 3), ref.blocktransp(w, 4, 5, 3, 3), "blocktransp")
    assert_exact(oracle.blocktransp(w, 4, 5, 3, 3, hwc=1), ref.blocktransp(w, 4, 5, 3, 3, hwc=1), "blocktransp hwc")


def test_pointwise(oracle, ref):
    rng = seeded(11)
    C, H, W = 8, 6, 5
    x = rng.standard_normal((C, H, W)).astype(np.float32); w = rng.standard_normal((C, C)).astype(np.float32)
    dy = rng.standard_normal((C, H, W)).astype(np.float32)
    r = ref.pw(x, w, dy, C, C, H, W)
    g = geom(C, H, W, C, 1)
    w4 = w.reshape(C, C, 1, 1)
    assert_close(oracle.conv2d_fw(x, w4, None, g), r["y"], TIGHT, "pw fw")
    assert_close(oracle.conv2d_wg(x, dy, g)[0].reshape(C, C), r["dw"], TIGHT, "pw wg")
    assert_close(oracle.conv2d_ig(dy, w4, g), r["dx"], TIGHT, "pw ig (C_in == C_out)")


def test_depthwise(oracle, ref):
    rng = seeded(12)
    g = geom(6, 9, 8, 6, 3)
    Ho, Wo = out_hw(g)
    x = rng.standard_normal((6, 9, 8)).astype(np.float32); w = rng.standard_normal((6, 3, 3)).astype(np.float32)
    dy = rng.standard_normal((6, Ho, Wo)).astype(np.float32)
    r = ref.dw(x, w, dy, g)
    assert_close(oracle.dw_fw(x, w, g), r["y"], TIGHT, "dw fw")
    assert_close(oracle.dw_wg(x, dy, g), r["dw"], TIGHT, "dw wg")
    assert_close(oracle.dw_ig(dy, w, g), r["dx"], TIGHT, "dw ig")
    g1 = geom(6, 9, 8, 6, 3, stride=2, pad=1)       # forward honours stride/pad in the reference
    assert_close(oracle.dw_fw(x, w, g1), ref.dw(x, w, np.zeros((6,) + out_hw(g1), np.float32), g1)["y"], TIGHT, "dw fw s2p1")


@pytest.mark.parametrize("inn,out", [(8, 8), (33, 17), (256, 256)])
def test_linear(oracle, ref, inn, out):
    rng = seeded(inn + out)
    W = (rng.standard_normal((out, inn)) / np.sqrt(inn)).astype(np.float32)
    x = rng.standard_normal(inn).astype(np.float32); dy = rng.standard_normal(out).astype(np.float32)
    r = ref.linear(W, x, dy)
    o = oracle.linear(W, x, dy)
    for k in ("y", "dW", "dx"):
        assert_exact(o[k], r[k].reshape(o[k].shape), "linear %s" % k)


@pytest.mark.parametrize("L,E,F,heads", [(10, 10, 160, 5), (16, 8, 16, 2), (24, 12, 32, 4)])
def test_mhsa(oracle, ref, L, E, F, heads):
    rng = seeded(L * 7 + F)
    x = rng.standard_normal((E, L)).astype(np.float32); dy = rng.standard_normal((E, L)).astype(np.float32)
    ws = [(rng.standard_normal((E, F)) / np.sqrt(E)).astype(np.float32) for _ in range(4)]
    bs = [(0.1 * rng.standard_normal(F)).astype(np.float32) for _ in range(3)]
    r = ref.mhsa(x, ws[0], ws[1], ws[2], bs[0], bs[1], bs[2], ws[3], dy, L, E, F, heads)
    o = oracle.mhsa(x, ws[0], ws[1], ws[2], bs[0], bs[1], bs[2], ws[3], dy, L, E, F, heads)
    for k in ("q", "k", "v", "softmax", "att", "y", "dwo", "datt", "dv", "dsoftmax", "dk", "dq", "dwq", "dwk", "dwv", "dx"):
        assert_close(o[k], r[k].reshape(o[k].shape), 5e-6, "mhsa %s" % k)


def test_activations_softmax(oracle, ref):
    rng = seeded(21)
    x = (3 * rng.standard_normal(1000)).astype(np.float32); dy = rng.standard_normal(1000).astype(np.float32)
    for i, kind in enumerate(("relu", "leakyrelu", "sigmoid")):
        r = ref.act(kind, x, dy, slope=0.01)
        y = oracle.act_fw(i, x, 0.01)
        assert_close(y, r["y"], TIGHT, kind)
        assert_close(oracle.act_bw(i, x, y, dy, 0.01), r["dx"], TIGHT, kind + " bw")
    assert_close(oracle.act_fw(3, x), ref.act("gelu", x, dy)["y"], TIGHT, "gelu")
    s = (2 * rng.standard_normal((12, 37))).astype(np.float32); ds = rng.standard_normal((12, 37)).astype(np.float32)
    r = ref.softmax(s, ds)
    out = oracle.softmax_fw(s)
    assert_close(out, r["out"], TIGHT, "softmax")
    assert_close(oracle.softmax_bw(out, ds), r["din"], TIGHT, "softmax bw")


def test_norms(oracle, ref):
    rng = seeded(31)
    C, H, W = 8, 4, 4
    x = rng.standard_normal((C, H, W)).astype(np.float32); dy = rng.standard_normal((C, H, W)).astype(np.float32)
    gb = rng.standard_normal(2 * C).astype(np.float32)
    r = ref.instnorm(x, gb, dy); o = oracle.instnorm(x, gb, dy)
    for k in ("y", "dx", "dgb", "mean", "var", "std"):
        assert_close(o[k], r[k].reshape(o[k].shape), TIGHT, "instnorm %s" % k)
    B = 2
    xb = rng.standard_normal((B, C, H, W)).astype(np.float32)
    assert_close(oracle.batchnorm_fw(xb, gb[:C], gb[C:], B, C, H * W, 1e-5), ref.batchnorm_fw(xb, gb[:C], gb[C:], B, C, H, W, 1e-5), TIGHT, "batchnorm")
    xl = rng.standard_normal((16, 16)).astype(np.float32); wl = rng.standard_normal(16).astype(np.float32); bl = rng.standard_normal(16).astype(np.float32)
    assert_close(oracle.layernorm_fw(xl, wl, bl, 16, 16, 1e-5), ref.layernorm_fw(xl, wl, bl, 16, 16, 1e-5), TIGHT, "layernorm")


def test_losses_sgd_residual_pool(oracle, ref):
    rng = seeded(41)
    y = rng.standard_normal(10).astype(np.float32); t = rng.standard_normal(10).astype(np.float32)
    lr_, dyr = ref.loss("MSELoss", y, t); lo, dyo = oracle.mse(y, t)
    assert_close(lo, lr_, TIGHT, "mse"); assert_close(dyo, dyr, TIGHT, "mse bw")
    onehot = np.zeros(10, np.float32); onehot[3] = 1
    lr_, dzr = ref.loss("CrossEntropyLoss", y, onehot); lo, dzo = oracle.ce(y, onehot)
    assert_close(lo, lr_, TIGHT, "ce"); assert_close(dzo, dzr, TIGHT, "ce bw")
    w = rng.standard_normal(100).astype(np.float32); g = rng.standard_normal(100).astype(np.float32)
    for lam in (0.0, 0.01):
        r = ref.sgd(w, g, 1e-2, lam); wo, go = oracle.sgd(w, g, 1e-2, lam)
        assert_exact(wo, r["w"], "sgd w"); assert_exact(go, r["g"], "sgd g")
    x = rng.standard_normal((4, 8, 8)).astype(np.float32); dyp = rng.standard_normal((4, 1, 1)).astype(np.float32)
    r = ref.avgpool(x, dyp, 8, 8, 1, 1); yo, dxo = oracle.avgpool(x, dyp, 8, 8, 1, 1)
    assert_close(yo, r["y"], TIGHT, "avgpool"); assert_close(dxo, r["dx"], TIGHT, "avgpool bw")
    dyp2 = rng.standard_normal((4, 4, 4)).astype(np.float32)
    r = ref.avgpool(x, dyp2, 2, 2, 2, 2); yo, dxo = oracle.avgpool(x, dyp2, 2, 2, 2, 2)
    assert_close(yo, r["y"], TIGHT, "avgpool 2x2"); assert_close(dxo, r["dx"], TIGHT, "avgpool 2x2 bw")


def test_index_helpers(oracle, ref):
    rng = seeded(51)
    x = rng.standard_normal((13, 15, 17)).astype(np.float32)
    for axes in ((2, 0, 1), (1, 0, 2), (0, 2, 1)):
        got = oracle.transpose(x, axes)
        assert_exact(got, np.ascontiguousarray(x.transpose(axes)), "transpose numpy")
        assert_exact(got, ref.transpose(x, axes), "transpose ref")
    m = rng.standard_normal((7, 12)).astype(np.float32)
    assert_exact(oracle.transpose(m, (1, 0)), ref.transpose_matrix(m), "transpose_matrix")
    a = rng.standard_normal((4, 1, 6)).astype(np.float32); b = rng.standard_normal((5, 1)).astype(np.float32)
    assert_exact(oracle.broadcast_add(a, b), ref.broadcast_add(a, b), "broadcast add")
    assert_exact(oracle.broadcast_add(a, b), (a + b).astype(np.float32), "broadcast add numpy")
    p = rng.standard_normal((3, 5, 6)).astype(np.float32)
    assert_exact(oracle.pad(p, 1, 1, 1, 1), ref.pad(p, 1, 1, 1, 1), "pad 1")
    assert_exact(oracle.pad(p, 2, 1, 0, 3), np.pad(p, ((0, 0), (0, 3), (2, 1))), "pad numpy")


MMB_SHAPES = [((3, 5, 7), (3, 7, 4)), ((2, 1, 6, 5), (3, 5, 8)), ((1, 4, 9), (2, 3, 1, 9, 2)), ((4, 6, 3), (1, 3, 5))]


@pytest.mark.parametrize("sa,sb", MMB_SHAPES)
def test_mm_broadcast_oracle_is_numpy_matmul_and_the_reference(oracle, reflib, pkg, sa, sb):
    """mm_broadcast: the oracle restates NumPy broadcasting; pinned against numpy.matmul and the reference's own C"""
    from abi_runner import AbiRunner
    rng = np.random.default_rng(sum(sa) + sum(sb))
    A = rng.standard_normal(sa).astype(np.float32); B = rng.standard_normal(sb).astype(np.float32)
    want = np.matmul(A.astype(np.float64), B.astype(np.float64))
    got = oracle.mm_broadcast(A, B)
    assert got.shape == want.shape
    assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max()
    ref = AbiRunner(pkg, reflib, is_ref=True).mm_broadcast(A, B)
    assert np.array_equal(ref, got), "same products in the same order: bit-identical"


def test_hwc_conv2d_layout_convention_of_the_reference(oracle, reflib, pkg):
    """HWC Conv2D: activations [H][W][C], weights [Cout][Hk][Wk][Cin].  Pinned on the reference's im2col forward (no
    padding, where that path is right): permuting its operands gives the CHW oracle's result."""
    from abi_runner import AbiRunner
    from golden_cases import geom
    g = geom(5, 9, 8, 6, 3, pad=0)
    rng = np.random.default_rng(21)
    x = rng.standard_normal((5, 9, 8)).astype(np.float32); w = rng.standard_normal((6, 5, 3, 3)).astype(np.float32)
    want = oracle.conv2d_fw(x, w, None, g)
    r = AbiRunner(pkg, reflib, is_ref=True)
    got = r.conv2d(np.ascontiguousarray(x.transpose(1, 2, 0)), np.ascontiguousarray(w.transpose(0, 2, 3, 1)), None, g, use_im2col=1, steps=("fw",), hwc=1)
    Ho, Wo = want.shape[1:]
    y = got["y"].reshape(-1)[:want.size].reshape(Ho, Wo, 6).transpose(2, 0, 1)
    assert np.abs(y - want).max() <= 1e-5 * np.abs(want).max()
