"""One list of seeded cases that drives three things:
  * tests/golden/make_golden.py runs each case through the reference's own C code and stores
    inputs + outputs as tests/golden/<name>.npz;
  * the CPU tests run the oracle restatement on the stored inputs and compare with the stored outputs;
  * the GPU tests run libtrainlib_b200 through the same ABI and compare with both.

A case is (name, make_inputs(rng) -> dict, run_abi(runner, inp) -> dict, run_oracle(oracle, inp) -> dict,
tolerance or None for bit-exact).  Output keys of run_abi and run_oracle match.
"""
import numpy as np

from oracle_bind import geom, out_hw

F = np.float32
CASES = []


def case(name, tol):
    def deco(cls):
        CASES.append((name, cls.inputs, cls.abi, cls.oracle, tol))
        return cls
    return deco


def _conv_inputs(g, bias=False):
    def make(rng):
        Ho, Wo = out_hw(g)
        d = dict(x=rng.uniform(-1, 1, (g["Cin"], g["Hin"], g["Win"])).astype(F),
                 w=rng.uniform(-1, 1, (g["Cout"], g["Cin"], g["Hk"], g["Wk"])).astype(F),
                 dy=rng.standard_normal((g["Cout"], Ho, Wo)).astype(F))
        if bias:
            d["bias"] = rng.standard_normal(g["Cout"]).astype(F)
        return d
    return make


def _conv_case(name, g, use_im2col, bias=False, ref_steps=("fw", "wg", "ig")):
    class C(object):
        inputs = staticmethod(_conv_inputs(g, bias))

        @staticmethod
        def abi(r, i):
            steps = ref_steps if r.is_ref else ("fw", "wg", "ig")
            out = r.conv2d(i["x"], i["w"], i["dy"], g, use_im2col=use_im2col if r.is_ref else 1, bias=i.get("bias"), steps=steps)
            if bias and (g["padU"] > 0 or use_im2col):
                # the reference's bias grad is the channel sum only on the unpadded naive path: with
                # padding it drops border pixels, on the im2col path it sums the wrong tensor
                # (lib/sources/pulp_conv2d_fp32.c:752,795)
                out.pop("db", None)
            if not bias:
                out.pop("db", None)
            return out

        @staticmethod
        def oracle(o, i):
            dw, db = o.conv2d_wg(i["x"], i["dy"], g, with_bias=bias)
            out = dict(y=o.conv2d_fw(i["x"], i["w"], i.get("bias"), g), dw=dw, dx=o.conv2d_ig(i["dy"], i["w"], g))
            if bias and g["padU"] == 0 and not use_im2col:
                out["db"] = db
            return out
    case(name, 1e-5)(C)


# reference test default: 8 -> 8 channels, 8x8, 3x3, no padding (tests/test_conv2d_fp32/Makefile:4-15), im2col path
_conv_case("conv2d_ref_default_im2col", geom(8, 8, 8, 8, 3), 1, bias=True)
_conv_case("conv2d_bias_naive", geom(8, 8, 8, 8, 3), 0, bias=True)
# config 1 shape: 3x3 s1 p1, 16 -> 32 channels, 32x32; padded WG/IG from the reference's naive path
_conv_case("conv2d_c1_3x3_p1", geom(16, 32, 32, 32, 3, pad=1), 0)
# stride-2 downsampling block (naive path; the im2col path rejects it)
_conv_case("conv2d_3x3_s2_p1", geom(6, 10, 10, 4, 3, stride=2, pad=1), 0)
_conv_case("conv2d_1x1_s2", geom(6, 10, 10, 9, 1, stride=2, pad=0), 0, ref_steps=("fw", "wg"))
_conv_case("conv2d_5x5_p2", geom(5, 9, 9, 7, 5, pad=2), 0)
_conv_case("conv2d_ragged", geom(3, 9, 7, 5, 3), 1)


@case("mm_17x13x9", None)
class _MM(object):
    @staticmethod
    def inputs(rng):
        return dict(A=rng.standard_normal((17, 13)).astype(F), B=rng.standard_normal((13, 9)).astype(F), Bt=rng.standard_normal((9, 13)).astype(F))

    @staticmethod
    def abi(r, i):
        return dict(c=r.mm(i["A"], i["B"], 17, 13, 9, 0), ct=r.mm(i["A"], i["Bt"], 17, 13, 9, 1, fn="mm_M"))

    @staticmethod
    def oracle(o, i):
        return dict(c=o.mm(i["A"], i["B"], 17, 13, 9, 0), ct=o.mm(i["A"], i["Bt"], 17, 13, 9, 1))


# the GPU sums in a different order, so the GPU comparison of this case uses a tolerance
MM_GPU_TOL = 1e-5


def _linear_case(name, inn, out):
    class C(object):
        @staticmethod
        def inputs(rng):
            return dict(W=(rng.standard_normal((out, inn)) / np.sqrt(inn)).astype(F), x=rng.standard_normal(inn).astype(F),
                        dy=rng.standard_normal(out).astype(F))

        @staticmethod
        def abi(r, i):
            res = r.linear(i["W"], i["x"], i["dy"])
            return dict(y=res["y"], dW=res["dW"], dx=res["dx"])

        @staticmethod
        def oracle(o, i):
            res = o.linear(i["W"], i["x"], i["dy"])
            return dict(y=res["y"], dW=res["dW"], dx=res["dx"])
    case(name, 1e-5)(C)


_linear_case("linear_8x8", 8, 8)            # reference test default
_linear_case("linear_33x17", 33, 17)
_linear_case("linear_256x256", 256, 256)    # smallest shape of the config-2 sweep


def _mhsa_case(name, L, E, Fd, heads):
    class C(object):
        @staticmethod
        def inputs(rng):
            d = dict(x=rng.standard_normal((E, L)).astype(F), dy=rng.standard_normal((E, L)).astype(F))
            for n in ("wq", "wk", "wv", "wo"):
                d[n] = (rng.standard_normal((E, Fd)) / np.sqrt(E)).astype(F)
            for n in ("bq", "bk", "bv"):
                d[n] = (0.1 * rng.standard_normal(Fd)).astype(F)
            return d

        @staticmethod
        def abi(r, i):
            return r.mhsa(i["x"], i["wq"], i["wk"], i["wv"], i["bq"], i["bk"], i["bv"], i["wo"], i["dy"], L, E, Fd, heads)

        @staticmethod
        def oracle(o, i):
            return o.mhsa(i["x"], i["wq"], i["wk"], i["wv"], i["bq"], i["bk"], i["bv"], i["wo"], i["dy"], L, E, Fd, heads)
    case(name, 1e-5)(C)


def _mobilebert_inputs(L, E, Kb, Fd, No):
    def make(rng):
        d = dict(x=rng.standard_normal((L, E)).astype(F), xb=rng.standard_normal((L, Kb)).astype(F), dy=rng.standard_normal((L, No)).astype(F))
        d["wq"] = (rng.standard_normal((Fd, Kb)) / np.sqrt(Kb)).astype(F); d["wk"] = (rng.standard_normal((Fd, Kb)) / np.sqrt(Kb)).astype(F)
        d["wv"] = (rng.standard_normal((Fd, E)) / np.sqrt(E)).astype(F); d["wo"] = (rng.standard_normal((No, Fd)) / np.sqrt(Fd)).astype(F)
        for n, m in (("bq", Fd), ("bk", Fd), ("bv", Fd), ("bo", No)):
            d[n] = (0.1 * rng.standard_normal(m)).astype(F)
        return d
    return make


def _mobilebert_case(name, L, E, Fd, heads):
    """forward of the MobileBERT inference attention (F = Kb = No) through the reference's own function, built with -DOPTIMIZE"""
    class C(object):
        inputs = staticmethod(_mobilebert_inputs(L, E, Fd, Fd, Fd))

        @staticmethod
        def abi(r, i):
            return r.mobilebert(i["x"], i["xb"], i["wq"], i["wk"], i["wv"], i["bq"], i["bk"], i["bv"], i["wo"], i["bo"], None, L, E, Fd, Fd, Fd, heads)

        @staticmethod
        def oracle(o, i):
            return o.mobilebert(i["x"], i["xb"], i["wq"], i["wk"], i["wv"], i["bq"], i["bk"], i["bv"], i["wo"], i["bo"], None, L, E, Fd, Fd, Fd, heads)
    case(name, 1e-5)(C)


_mobilebert_case("mhsa_mobilebert_L24_E20_F32_h4", 24, 20, 32, 4)
_mobilebert_case("mhsa_mobilebert_L37_E48_F40_h5", 37, 48, 40, 5)
_mhsa_case("mhsa_ref_default", 10, 10, 160, 5)      # tests/test_mhsa_fp32/Makefile:4-7
_mhsa_case("mhsa_L24_E12_F32_h4", 24, 12, 32, 4)


@case("pointwise_8ch", 1e-5)
class _PW(object):
    @staticmethod
    def inputs(rng):
        return dict(x=rng.standard_normal((8, 6, 5)).astype(F), w=rng.standard_normal((8, 8)).astype(F), dy=rng.standard_normal((8, 6, 5)).astype(F))

    @staticmethod
    def abi(r, i):
        return r.pw(i["x"], i["w"], i["dy"], 8, 8, 6, 5)

    @staticmethod
    def oracle(o, i):
        g = geom(8, 6, 5, 8, 1)
        w4 = i["w"].reshape(8, 8, 1, 1)
        return dict(y=o.conv2d_fw(i["x"], w4, None, g), dw=o.conv2d_wg(i["x"], i["dy"], g)[0].reshape(8, 8), dx=o.conv2d_ig(i["dy"], w4, g))


@case("depthwise_6ch", 1e-5)
class _DW(object):
    g = geom(6, 9, 8, 6, 3)

    @staticmethod
    def inputs(rng):
        return dict(x=rng.standard_normal((6, 9, 8)).astype(F), w=rng.standard_normal((6, 3, 3)).astype(F), dy=rng.standard_normal((6, 7, 6)).astype(F))

    @staticmethod
    def abi(r, i):
        return r.dw(i["x"], i["w"], i["dy"], _DW.g)

    @staticmethod
    def oracle(o, i):
        return dict(y=o.dw_fw(i["x"], i["w"], _DW.g), dw=o.dw_wg(i["x"], i["dy"], _DW.g), dx=o.dw_ig(i["dy"], i["w"], _DW.g))


@case("activations", 1e-5)
class _ACT(object):
    @staticmethod
    def inputs(rng):
        return dict(x=(3 * rng.standard_normal(1000)).astype(F), dy=rng.standard_normal(1000).astype(F))

    @staticmethod
    def abi(r, i):
        out = {}
        for kind in ("relu", "leakyrelu", "sigmoid"):
            res = r.act(kind, i["x"], i["dy"], slope=0.01)
            out[kind] = res["y"]; out[kind + "_bw"] = res["dx"]
        out["gelu"] = r.act("gelu", i["x"], i["dy"])["y"]
        return out

    @staticmethod
    def oracle(o, i):
        out = {}
        for k, kind in enumerate(("relu", "leakyrelu", "sigmoid")):
            y = o.act_fw(k, i["x"], 0.01)
            out[kind] = y; out[kind + "_bw"] = o.act_bw(k, i["x"], y, i["dy"], 0.01)
        out["gelu"] = o.act_fw(3, i["x"])
        return out


@case("softmax_12x37", 1e-5)
class _SM(object):
    @staticmethod
    def inputs(rng):
        return dict(s=(2 * rng.standard_normal((12, 37))).astype(F), ds=rng.standard_normal((12, 37)).astype(F))

    @staticmethod
    def abi(r, i):
        return r.softmax(i["s"], i["ds"])

    @staticmethod
    def oracle(o, i):
        out = o.softmax_fw(i["s"])
        return dict(out=out, din=o.softmax_bw(out, i["ds"]))


@case("norms", 1e-5)
class _NORM(object):
    @staticmethod
    def inputs(rng):
        return dict(x=rng.standard_normal((8, 4, 4)).astype(F), dy=rng.standard_normal((8, 4, 4)).astype(F), gb=rng.standard_normal(16).astype(F),
                    xb=rng.standard_normal((2, 4, 4, 4)).astype(F), xl=rng.standard_normal((16, 16)).astype(F),
                    wl=rng.standard_normal(16).astype(F), bl=rng.standard_normal(16).astype(F))

    @staticmethod
    def abi(r, i):
        res = r.instnorm(i["x"], i["gb"], i["dy"])
        out = {"in_" + k: res[k] for k in ("y", "dx", "dgb", "mean", "var", "std")}
        out["bn_y"] = r.batchnorm_fw(i["xb"], i["gb"][:4], i["gb"][4:8], 2, 4, 4, 4, 1e-5)     # tests/test_batchnorm_fp32/Makefile:4-8
        out["ln_y"] = r.layernorm_fw(i["xl"], i["wl"], i["bl"], 16, 16, 1e-5)
        return out

    @staticmethod
    def oracle(o, i):
        res = o.instnorm(i["x"], i["gb"], i["dy"])
        out = {"in_" + k: res[k] for k in ("y", "dx", "dgb", "mean", "var", "std")}
        out["bn_y"] = o.batchnorm_fw(i["xb"], i["gb"][:4], i["gb"][4:8], 2, 4, 16, 1e-5)
        out["ln_y"] = o.layernorm_fw(i["xl"], i["wl"], i["bl"], 16, 16, 1e-5)
        return out


@case("losses_sgd_pool_residual", 1e-5)
class _MISC(object):
    @staticmethod
    def inputs(rng):
        t = np.zeros(10, F); t[3] = 1
        return dict(y=rng.standard_normal(10).astype(F), t=rng.standard_normal(10).astype(F), onehot=t,
                    w=rng.standard_normal(100).astype(F), g=rng.standard_normal(100).astype(F),
                    x=rng.standard_normal((4, 8, 8)).astype(F), dyp=rng.standard_normal((4, 1, 1)).astype(F), dyp2=rng.standard_normal((4, 4, 4)).astype(F),
                    skip=rng.standard_normal(300).astype(F), lout=rng.standard_normal(300).astype(F), dout=rng.standard_normal(300).astype(F),
                    dskip0=rng.standard_normal(300).astype(F))

    @staticmethod
    def abi(r, i):
        out = {}
        out["mse"], out["mse_dy"] = r.loss("MSELoss", i["y"], i["t"])
        out["ce"], out["ce_dz"] = r.loss("CrossEntropyLoss", i["y"], i["onehot"])
        s = r.sgd(i["w"], i["g"], 1e-2, 0.0); out["sgd_w"] = s["w"]
        s = r.sgd(i["w"], i["g"], 1e-2, 0.01); out["sgd_w_decay"] = s["w"]; out["sgd_g_decay"] = s["g"]
        p = r.avgpool(i["x"], i["dyp"], 8, 8, 1, 1); out["gap_y"] = p["y"]; out["gap_dx"] = p["dx"]
        p = r.avgpool(i["x"], i["dyp2"], 2, 2, 2, 2); out["pool_y"] = p["y"]; out["pool_dx"] = p["dx"]
        res = r.residual(i["skip"], i["lout"], i["dout"], i["dskip0"])
        out["res_out"] = res["out"]; out["res_dskip"] = res["dskip"]; out["res_dlout"] = res["dlout"]
        return {k: np.asarray(v, F) for k, v in out.items()}

    @staticmethod
    def oracle(o, i):
        out = {}
        out["mse"], out["mse_dy"] = o.mse(i["y"], i["t"])
        out["ce"], out["ce_dz"] = o.ce(i["y"], i["onehot"])
        out["sgd_w"], _ = o.sgd(i["w"], i["g"], 1e-2, 0.0)
        out["sgd_w_decay"], out["sgd_g_decay"] = o.sgd(i["w"], i["g"], 1e-2, 0.01)
        out["gap_y"], out["gap_dx"] = o.avgpool(i["x"], i["dyp"], 8, 8, 1, 1)
        out["pool_y"], out["pool_dx"] = o.avgpool(i["x"], i["dyp2"], 2, 2, 2, 2)
        out["res_out"] = (i["skip"] + i["lout"]).astype(F); out["res_dskip"] = (i["dout"] + i["dskip0"]).astype(F); out["res_dlout"] = i["dout"].copy()
        return {k: np.asarray(v, F) for k, v in out.items()}


@case("index_helpers", None)
class _IDX(object):
    g0 = geom(4, 7, 6, 5, 3)
    g1 = geom(4, 7, 6, 5, 3, pad=1)

    @staticmethod
    def inputs(rng):
        return dict(x=rng.standard_normal((4, 7, 6)).astype(F), dy=rng.standard_normal((5, 5, 4)).astype(F), w=rng.standard_normal((5, 4, 3, 3)).astype(F),
                    t3=rng.standard_normal((13, 15, 17)).astype(F), m=rng.standard_normal((7, 12)).astype(F),
                    a=rng.standard_normal((4, 1, 6)).astype(F), b=rng.standard_normal((5, 1)).astype(F), p=rng.standard_normal((3, 5, 6)).astype(F))

    @staticmethod
    def abi(r, i):
        return dict(i2r=r.im2row(i["x"], _IDX.g0, mod=0), i2r_pad=r.im2row(i["x"], _IDX.g1, mod=0), i2r_ig=r.im2row(i["dy"], _IDX.g0, mod=1),
                    i2c=r.im2row(i["x"], _IDX.g0, mod=0, fn="pulp_im2col_fp32"),
                    bt=r.blocktransp(i["w"], 4, 5, 3, 3), bt_hwc=r.blocktransp(i["w"], 4, 5, 3, 3, hwc=1),
                    tr=r.transpose(i["t3"], (2, 0, 1)), tr2=r.transpose(i["t3"], (1, 0, 2)), trm=r.transpose_matrix(i["m"]),   # tests/test_transpose/Makefile
                    badd=r.broadcast_add(i["a"], i["b"]), pad=r.pad(i["p"], 1, 1, 1, 1))

    @staticmethod
    def oracle(o, i):
        return dict(i2r=o.im2row(i["x"], 4, 7, 6, 3, 3, 5, 4, 1, 1, 0, 0), i2r_pad=o.im2row(i["x"], 4, 7, 6, 3, 3, 7, 6, 1, 1, 1, 1),
                    i2r_ig=o.im2row(i["dy"], 5, 7, 6, 3, 3, 5, 4, 1, 1, 0, 0, mode_ig=1), i2c=o.im2row(i["x"], 4, 7, 6, 3, 3, 5, 4, 1, 1, 0, 0, transposed=1),
                    bt=o.blocktransp(i["w"], 4, 5, 3, 3), bt_hwc=o.blocktransp(i["w"], 4, 5, 3, 3, hwc=1),
                    tr=o.transpose(i["t3"], (2, 0, 1)), tr2=o.transpose(i["t3"], (1, 0, 2)), trm=o.transpose(i["m"], (1, 0)),
                    badd=o.broadcast_add(i["a"], i["b"]), pad=o.pad(i["p"], 1, 1, 1, 1))


def family_oracle(i, with_shift=True):
    """numpy float32 restatement of the element-wise family, loop for loop where a sum's order matters
    [ref: lib/sources/pulp_losses_fp32.c:140-365, pulp_pooling_fp32.c:123-237, pulp_nonorm_fp32.c:30-58,
    pulp_rmsnorm_fp32.c:29-95, pulp_act_fp32.c:651-712, pulp_train_utils_fp32.c:987-1264, :1730-1756]"""
    f = np.float32
    r = {}
    y, t = i["y"].ravel(), i["t"].ravel(); n = y.size
    mean = f(1.0) / f(n)
    loss = f(0)
    for k in range(n):
        loss = f(loss + f(mean * abs(f(t[k] - y[k]))))
    d = (y - t).astype(f)
    r["l1"] = np.array([loss], f); r["l1_dy"] = (np.sign(d) * mean).astype(f).reshape(i["y"].shape)
    c = f(f(i["alpha"][0]) * np.abs(d).max())
    loss = f(0)
    for k in range(n):
        v = abs(d[k])
        loss = f(loss + (v if v < c else f(f(f(v * v) - f(c * c)) / f(f(2) * c))))
    r["berhu"] = np.array([f(loss * mean)], f)
    r["berhu_dy"] = np.where(np.abs(d) < c, np.sign(d) * mean, f(mean) * d / c).astype(f).reshape(i["y"].shape)
    for tag, x, g, (Hk, Wk, sh, sw) in (("mp2", i["px"], i["pdy2"], (2, 2, 2, 2)), ("mp3", i["pxt"], i["pdy3"], (3, 3, 1, 1))):
        C, H, W = x.shape
        Ho, Wo = (H - Hk + sh) // sh, (W - Wk + sw) // sw
        out = np.zeros((C, Ho, Wo), f); dx = np.zeros_like(x)
        for ch in range(C):
            for ho in range(Ho):
                for wo in range(Wo):
                    win = x[ch, ho * sh:ho * sh + Hk, wo * sw:wo * sw + Wk]
                    out[ch, ho, wo] = win.max()
                    a, b = np.unravel_index(np.argmax(win), win.shape)         # first maximum in row-major order
                    dx[ch, ho * sh + a, wo * sw + b] += g[ch, ho, wo]
        r[tag + "_y"] = out; r[tag + "_dx"] = dx
    r["nonorm"] = (i["nx"] * i["nw"][None, :]).astype(f) + i["nb"][None, :]
    v, w = i["v"], i["w"]
    r["wscale"] = (w * (f(0.37) * v).astype(f)).astype(f)
    ss = f(0)
    for k in range(v.size):
        ss = f(ss + f(v[k] * v[k]))
    r["sumsq"] = np.array([ss], f)
    sf = f(f(1) / np.sqrt(f(f(ss / f(v.size)) + f(1e-5)), dtype=f))
    r["rmsnorm"] = (w * (sf * v).astype(f)).astype(f)
    sig = (f(1) / (f(1) + np.exp(-v, dtype=f))).astype(f)
    r["swiglu"] = ((v * sig).astype(f) * w).astype(f)
    e = np.exp((v - v.max()).astype(f), dtype=f)
    es = f(0)
    for k in range(v.size):
        es = f(es + e[k])
    r["vsoftmax"] = (e / es).astype(f)
    r["vmax"] = np.array([v.max()], f); r["vexp"] = e; r["vexp_sum"] = np.array([es], f)
    r["vdiv"] = (v / f(1.7)).astype(f)
    A, B = i["A"], i["B"]
    S = np.zeros(A.shape[0], f)
    for row in range(A.shape[0]):
        acc = f(0)
        for col in range(A.shape[1]):
            acc = f(acc + f(A[row, col] * B[row, col]))
        S[row] = acc
    r["op1"] = S; r["op2"] = ((A - S[:, None]).astype(f) * B).astype(f)
    if with_shift:
        sq = i["sq"]; x = (sq.max(axis=1)[:, None] - sq).astype(f)
        x2 = (x * x).astype(f); x3 = (x2 * x).astype(f); x4 = (x3 * x).astype(f); x5 = (x4 * x).astype(f)
        p = f(1.0) - (f(0.6931471805599453) * x).astype(f)
        p = p + ((f(0.5) * x2).astype(f) * f(0.4804530139182014)).astype(f)
        p = p - ((f(0.16) * x3).astype(f) * f(0.3330246519889294)).astype(f)
        p = p + ((f(0.0416) * x4).astype(f) * f(0.2308350985830834)).astype(f)
        p = p - ((f(0.008) * x5).astype(f) * f(0.1600026977571413)).astype(f)
        o = np.where(x >= f(3.14), f(0), p).astype(f)
        r["shift"] = o
        su = np.zeros(o.shape[0], f)
        for row in range(o.shape[0]):
            acc = f(0)
            for col in range(o.shape[1]):
                acc = f(acc + o[row, col])
            su[row] = acc
        r["shift_sum"] = su
    return r


@case("elementwise_family", 1e-5)
class _Family(object):
    @staticmethod
    def inputs(rng):
        g = lambda *s: rng.standard_normal(s).astype(F)
        pxt = np.round(2 * g(3, 7, 6)).astype(F) / 2                       # many equal values: ties inside overlapping windows
        return dict(y=g(9, 7), t=g(9, 7), alpha=np.array([0.2], F), px=g(3, 8, 6), pdy2=g(3, 4, 3), pxt=pxt, pdy3=g(3, 5, 4),
                    nx=g(11, 24), nw=g(24), nb=g(24), v=(1.5 * g(203)).astype(F), w=g(203), A=g(7, 33), B=g(7, 33), sq=(2 * g(12, 12)).astype(F))

    @staticmethod
    def abi(r, i):
        return r.family(i)

    @staticmethod
    def oracle(o, i):
        return family_oracle(i)


def case_seed(name):
    return sum(ord(c) * (k + 1) for k, c in enumerate(name)) % (2 ** 31)
