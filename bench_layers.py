"""Single-layer workloads of bench.py: config 1 (one Conv2D training step) and config 3 (multi-head self-attention
forward + backward), both at batch 1 through the reference's own entry points.  Each class offers the device-resident
step (`step_device`) and the host-pointer step (`step_host`) that bench.py times."""
import ctypes

import numpy as np

F = np.float32


class _Layer(object):
    use_graph = True

    def __init__(self, pkg, lib):
        self.pkg, self.lib = pkg, lib
        self.keep = pkg.Keep()

    def l2_flush(self):
        self.lib.trainlib_memset(self.flush.ptr, 1, self.flush.nbytes)

    def _dev(self, arrays):
        """device copies of the arrays (zeros where an int element count is given)"""
        out = []
        for a in arrays:
            out.append(self.pkg.DeviceBuffer(self.lib, a) if isinstance(a, np.ndarray) else self.pkg.DeviceBuffer(self.lib, nbytes=4 * int(a)))
            if not isinstance(a, np.ndarray):
                out[-1].zero()
        return out

    def _host(self, lib, arrays):
        from bench import pinned_like
        out = []
        for a in arrays:
            a = a if isinstance(a, np.ndarray) else np.zeros(int(a), F)
            out.append(pinned_like(self.pkg, lib, a) if hasattr(lib, "trainlib_malloc_host") else a.copy())
        return out


class ConvStep(_Layer):
    """config 1: Conv2D 3x3, stride 1, pad 1, CI = 16, 32 x 32, CO = 32; x, W ~ U(-1, 1), bias 0, dY ~ N(0, 1);
    FW + WG + IG + one SGD update with lr 1e-3."""
    name = "c1_conv2d_16x32x32_to_32_k3_fw_wg_ig_sgd_batch1"
    CI, H, CO, K = 16, 32, 32, 3

    def __init__(self, pkg, lib):
        _Layer.__init__(self, pkg, lib)
        self.flops = 3 * 2.0 * self.CO * self.CI * 9 * self.H * self.H
        self.bytes = 4.0 * (2 * self.CI * self.H ** 2 + 2 * self.CO * self.H ** 2 + 5 * self.CO * self.CI * 9)

    def _tensors(self):
        rng = np.random.default_rng(1)
        x = rng.uniform(-1, 1, (self.CI, self.H, self.H)).astype(F); w = rng.uniform(-1, 1, (self.CO, self.CI, 3, 3)).astype(F)
        dy = rng.standard_normal((self.CO, self.H, self.H)).astype(F)
        # x, dx, w, dw, y, dy, one (bias / scratch stand-in)
        return [x, x.size, w, w.size, dy.size, dy, 1]

    def _args(self, p):
        pk, k = self.pkg, self.keep
        x, dx, w, dw, y, dy, one = p
        conv = pk.make_args(k, "Conv2D_args", input=pk.make_blob(k, x, dx, C=self.CI, H=self.H, W=self.H),
                            coeff=pk.make_blob(k, w, dw, C=self.CI, H=3, W=3, dim=self.CO * self.CI * 9), bias=pk.make_blob(k, one, one),
                            output=pk.make_blob(k, y, dy, C=self.CO, H=self.H, W=self.H), Lpad=1, Rpad=1, Upad=1, Dpad=1, stride_h=1, stride_w=1,
                            i2c_buffer=one, bt_buffer=one, skip_wg_grad=0, skip_in_grad=0, HWC=0, USE_BIASES=0, USE_IM2COL=0, USE_DMA_IM2COL=0,
                            opt_matmul_type_fw=0, opt_matmul_type_wg=0, opt_matmul_type_ig=0)
        wb = pk.make_blob(k, w, dw, dim=self.CO * self.CI * 9, W=self.CO * self.CI * 9)
        opt = pk.make_args(k, "optim_args", weights=wb, biases=wb, learning_rate=1e-3, weight_decay_lambda=0.0, use_biases=0)
        return conv, opt

    def setup_device(self):
        self.dev = self._dev(self._tensors())
        self.args_dev = self._args([b.ptr for b in self.dev])
        self.flush = self.pkg.DeviceBuffer(self.lib, nbytes=256 << 20)

    def _step(self, lib, args):
        conv, opt = args
        lib.pulp_conv2d_fp32_fw_cl(ctypes.byref(conv))
        lib.pulp_conv2d_fp32_bw_param_grads_cl(ctypes.byref(conv))
        lib.pulp_conv2d_fp32_bw_input_grads_cl(ctypes.byref(conv))
        lib.pulp_gradient_descent_fp32(ctypes.byref(opt))

    def step_device(self):
        self._step(self.lib, self.args_dev)

    def setup_host(self, lib):
        self.host = self._host(lib, self._tensors())
        self.args_host = self._args(self.host)
        n = lambda i: self.host[i].nbytes
        # per call the library uploads what the call reads and downloads what it writes
        self.h2d = (n(0) + n(2)) + (n(0) + n(5)) + (n(5) + n(2)) + 2 * n(2)
        self.d2h = n(4) + n(3) + n(1) + n(2)

    def step_host(self, lib):
        self._step(lib, self.args_host)

    def metric(self, ms):
        return {"metric": "train_step_tflops", "unit": "TFLOP/s", "value": self.flops / (ms * 1e-3) / 1e12}

    def roofline(self, ms, pk):
        tf = self.flops / (ms * 1e-3) / 1e12
        peak = pk["bf16_tflops_sustained"] / 6.0
        return {"bound": "tensor", "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak, "traffic": None, "peak_source": pk["source"],
                "kernel": "conv FW + WG + IG + SGD (whole step, 7 launches)", "algorithmic_flops": self.flops, "algorithmic_bytes": self.bytes,
                "us_per_step": 1e3 * ms, "hbm_frac": self.bytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"],
                "peak_note": "3xTF32-effective fp32 peak = measured sustained bf16 / 6; at 28 MFLOP and 0.5 MB the step is bound by launch latency, "
                             "neither by the tensor cores nor by HBM"}


class MhsaStep(_Layer):
    """config 3: multi-head self-attention, fp32, L = E = F = 256, 4 heads of 64; x ~ N(0, 1), W ~ N(0, 1/E), biases 0,
    dY ~ N(0, 1); forward + backward."""
    name = "c3_mhsa_L256_E256_h4_fw_bw_batch1"
    L = E = Fd = 256
    HEADS = 4

    def __init__(self, pkg, lib):
        _Layer.__init__(self, pkg, lib)
        L, E, Fd = self.L, self.E, self.Fd
        fw = 2.0 * (3 * L * E * Fd + 2 * L * L * Fd + L * Fd * E)
        self.flops = 3 * fw
        self.bytes = 4.0 * (3 * 4 * E * Fd + 2 * (2 * E * L + 4 * Fd * L * 2 + 2 * self.HEADS * L * L))

    def _tensors(self):
        rng = np.random.default_rng(3)
        L, E, Fd, h = self.L, self.E, self.Fd, self.HEADS
        x = rng.standard_normal((E, L)).astype(F); dy = rng.standard_normal((E, L)).astype(F)
        ws = [(rng.standard_normal((E, Fd)) / np.sqrt(E)).astype(F) for _ in range(4)]
        zb = np.zeros(Fd, F)
        tmax = max(L * L, E * Fd, L * Fd, E * L)
        #        0  1      2..5          6..9                        10..12        13..15
        return ([x, E * L] + ws + [Fd * E, Fd * E, Fd * E, E * Fd] + [zb, zb, zb] + [Fd, Fd, Fd] +
                # 16..19 q k v att, 20..23 their gradients, 24 softmax, 25 its gradient, 26 y, 27 dy, 28 temp, 29 grad, 30 maxes, 31 sums
                [Fd * L] * 8 + [h * L * L, h * L * L, E * L, dy, tmax, L * L, L, L])

    def _args(self, p):
        pk, k = self.pkg, self.keep
        L, E, Fd, h = self.L, self.E, self.Fd, self.HEADS
        b = lambda d, g, H, W: pk.make_blob(k, d, g, C=1, H=H, W=W)
        return pk.make_args(k, "Mhsa_args", input=b(p[0], p[1], L, E), n_heads=h, output=b(p[26], p[27], L, E),
                            coeff_in_q=b(p[2], p[6], Fd, E), coeff_in_k=b(p[3], p[7], Fd, E), coeff_in_v=b(p[4], p[8], Fd, E), coeff_out=b(p[5], p[9], E, Fd),
                            bias_in_q=pk.make_blob(k, p[10], p[13], dim=Fd, W=Fd), bias_in_k=pk.make_blob(k, p[11], p[14], dim=Fd, W=Fd),
                            bias_in_v=pk.make_blob(k, p[12], p[15], dim=Fd, W=Fd),
                            q=b(p[16], p[20], L, Fd), k=b(p[17], p[21], L, Fd), v=b(p[18], p[22], L, Fd), attention_map=b(p[19], p[23], L, Fd),
                            temp_buffer=p[28], grad=p[29], softmax_buffer=b(p[24], p[25], h, L * L), maxes=p[30], sums=p[31],
                            opt_matmul_type_fw=0, opt_matmul_type_wg=0, opt_matmul_type_ig=0)

    def setup_device(self):
        self.dev = self._dev(self._tensors())
        self.args_dev = self._args([b.ptr for b in self.dev])
        self.flush = self.pkg.DeviceBuffer(self.lib, nbytes=256 << 20)

    def _step(self, lib, args, dx):
        lib.pulp_mhsa_fp32_fw_cl(ctypes.byref(args))
        dx()                                         # the backward accumulates into input.diff: the caller zeroes it
        lib.pulp_mhsa_fp32_bw_cl(ctypes.byref(args))

    def step_device(self):
        self._step(self.lib, self.args_dev, self.dev[1].zero)

    def setup_host(self, lib):
        self.host = self._host(lib, self._tensors())
        self.args_host = self._args(self.host)
        n = lambda i: self.host[i].nbytes
        w4 = sum(n(i) for i in (2, 3, 4, 5))
        self.h2d = (n(0) + w4) + (n(0) + w4 + n(27) + 4 * n(16) + n(24) + n(1))
        self.d2h = (n(26) + 4 * n(16) + n(24)) + (n(1) + w4 + 4 * n(16) + n(25))

    def step_host(self, lib):
        self._step(lib, self.args_host, lambda: self.host[1].fill(0))

    def metric(self, ms):
        return {"metric": "fw_bw_tflops", "unit": "TFLOP/s", "value": self.flops / (ms * 1e-3) / 1e12}

    def roofline(self, ms, pk):
        tf = self.flops / (ms * 1e-3) / 1e12
        return {"bound": "ffma", "achieved": tf, "peak": 72.8, "unit": "TFLOP/s", "frac": tf / 72.8, "traffic": None, "peak_source": pk["source"],
                "kernel": "attention forward + backward: 11 launches (fused score-softmax-value kernel and its two backward kernels, projections and weight gradients as strided FFMA GEMMs)", "algorithmic_flops": self.flops,
                "algorithmic_bytes": self.bytes, "us_per_step": 1e3 * ms,
                "peak_note": "FFMA peak measured on this part (125 MAC/clk/SM); the 256^3 products stay on the FFMA tiles because their summation "
                             "order keeps the backward inside 1e-5 of the reference"}


class _LnArgs(ctypes.Structure):
    """struct trainlib_layernorm_args of include/trainlib_b200.h"""
    _fields_ = [(n, ctypes.c_void_p) for n in ("x", "weight", "bias", "output", "eps")] + [("size", ctypes.c_int), ("step_size", ctypes.c_int)] + \
               [(n, ctypes.c_void_p) for n in ("dy", "dx", "dweight", "dbias")]


class MobileBertBlock(_Layer):
    """config 4: MobileBERT-style encoder block at batch 1, forward + full backward + MSE loss, as a sequence of the
    library's entry points on device-resident tensors (tokens row-major, [L x features]):

        x1 = LN(X Wbi)                       bottleneck 512 -> 128
        x2 = LN(x1 + MHSA(x1))               L = 128, E = F = 128, 4 heads of 32 (the MobileBERT attention entry points, token-major)
        x  = LN(x + GELU(x W1) W2)   x 4     feed-forward 128 -> 512 -> 128
        Y  = LN(X + x Wbo)                   128 -> 512
        loss = MSE(Y, target)

    Linear layers are `mm` products (no biases), their backward two more products plus one transpose; weights ~ N(0, 0.02),
    input and target ~ N(0, 1), layer-norm weights 1 + N(0, 0.02), biases N(0, 0.02).  `half` selects the fp16 twins."""
    L, H, B, HEADS, NFFN, FF = 128, 512, 128, 4, 4, 512
    LOSS_SCALE = 1024.0
    no_reference = "the reference has no backward for layer norm and GELU, so it cannot run this block's training step"

    def __init__(self, pkg, lib, half=True):
        _Layer.__init__(self, pkg, lib)
        self.half = half
        self.dt = np.float16 if half else np.float32
        self.es = 2 if half else 4
        self.sfx = "_fp16" if half else ""
        self.name = "c4_mobilebert_block_L128_h512_b128_4ffn_%s_fw_bw_batch1" % ("fp16" if half else "fp32")
        L, H, B, FF = self.L, self.H, self.B, self.FF
        macs = L * H * B + (4 * L * B * B + 2 * L * L * B) + self.NFFN * 2 * L * B * FF + L * B * H
        self.flops = 3 * 2.0 * macs
        self.bufs, self.fw, self.bw_flat = {}, [], []
        self.params = []
        self.use_graph = True

    # ---------------------------------------------------------------- tensors
    def _t(self, name, shape, init=None):
        """device tensor + gradient; `init` = host array for the data"""
        n = int(np.prod(shape))
        if init is not None:
            init = init.astype(np.float16).astype(F)          # the fp32 twin of the block starts from the same fp16-representable values
        d = self.pkg.DeviceBuffer(self.lib, init.astype(self.dt)) if init is not None else self.pkg.DeviceBuffer(self.lib, nbytes=n * self.es)
        g = self.pkg.DeviceBuffer(self.lib, nbytes=n * self.es)
        if init is None:
            d.zero()
        g.zero()
        self.bufs[name] = (d, g, tuple(shape))
        return name

    def d(self, n): return self.bufs[n][0].ptr
    def g(self, n): return self.bufs[n][1].ptr
    def shape(self, n): return self.bufs[n][2]

    def get(self, name, grad=False):
        d, g, shape = self.bufs[name]
        return (g if grad else d).download(self.dt, shape).astype(np.float32)

    def _blob(self, n, H=1, W=None):
        size = int(np.prod(self.shape(n)))
        return self.pkg.make_blob(self.keep, self.d(n), self.g(n), C=1, H=H, W=W if W is not None else size, dim=size, half=self.half)

    def _call(self, lst, fn, args):
        lst.append((getattr(self.lib, fn), args))

    # ---------------------------------------------------------------- layers (each appends forward and backward calls)
    def _mm(self, lst, A, B, C, N, K, M, trans_B):
        a = self.pkg.make_args(self.keep, "matMul_args" + self.sfx, A=A, B=B, C=C, N=N, K=K, M=M, trans_B=trans_B, USE_BIASES=0)
        self._call(lst, "mm" + self.sfx, a)

    def _transpose(self, lst, src, dst, N, M):
        a = self.pkg.make_args(self.keep, "transp_args" + self.sfx, in_matrix=src, out_matrix=dst, N=N, M=M)
        self._call(lst, "transpose_matrix" + self.sfx, a)

    def linear(self, x, w, y):
        L, K = self.shape(x); M = self.shape(w)[1]
        self._mm(self.fw, self.d(x), self.d(w), self.d(y), L, K, M, 0)
        bw = []
        self._mm(bw, self.g(y), self.d(w), self.g(x), L, M, K, 1)                 # dX = dY W^T
        xt = self._t(x + "_T_for_" + w, (K, L))
        self._transpose(bw, self.d(x), self.d(xt), L, K)
        self._mm(bw, self.d(xt), self.g(y), self.g(w), K, L, M, 0)                # dW = X^T dY
        return bw

    def layernorm(self, x, w, b, y):
        rows, width = self.shape(x)
        a = _LnArgs()
        a.x, a.weight, a.bias, a.output, a.eps = self.d(x), self.d(w), self.d(b), self.d(y), self.eps_host.ctypes.data
        a.size, a.step_size = rows * width, width
        a.dy, a.dx, a.dweight, a.dbias = self.g(y), self.g(x), self.g(w), self.g(b)
        self.keep.hold(a)
        self._call(self.fw, "trainlib_layernorm_fp16_fw_cl" if self.half else "pulp_layerNorm_fp32_fw_cl", a)
        bw = []
        self._call(bw, "trainlib_layernorm_fp16_bw_cl" if self.half else "trainlib_layernorm_fp32_bw_cl", a)
        return bw

    def gelu(self, x, y):
        n = int(np.prod(self.shape(x)))
        a = self.pkg.make_args(self.keep, "act_args" + self.sfx, input=self._blob(x), output=self._blob(y), H=1, W=n)
        self._call(self.fw, "pulp_gelu_fp16_fw_cl" if self.half else "pulp_gelu_tanh_approx_fp32_fw_cl", a)
        bw = []
        self._call(bw, "trainlib_gelu_fp16_bw_cl" if self.half else "trainlib_gelu_fp32_bw_cl", a)
        return bw

    def residual(self, skip, lout, out):
        """out = skip + lout.  Backward in two parts: `copy` (lout.diff = out.diff) runs before the branch's backward, `add`
        (skip.diff += out.diff) after the branch has written skip.diff."""
        a = self.pkg.make_args(self.keep, "SkipConn_args" + self.sfx, skip=self._blob(skip), lout=self._blob(lout), output=self._blob(out), skip_in_grad=0)
        r = "fp16" if self.half else "fp32"
        self._call(self.fw, "pulp_residualconn_%s_fw" % r, a)
        copy, add = [], []
        self._call(copy, "pulp_residualconn_%s_bw" % r, a)
        self._call(add, "pulp_sumnode_%s_bw" % r, a)
        return copy, add

    def mhsa(self, x, y):
        """x, y: [L x E] row-major (token-major), which is what the MobileBERT attention entry points take: the block's
        bottleneck activation is both `input` (source of V) and `input_bn` (source of Q and K); no transposes around the call.
        Wq, Wk, Wv, Wo are F x E row-major ([output feature][input feature]); all four biases are zero tensors."""
        L, E = self.shape(x); Fd, h = E, self.HEADS
        names = {}
        for n, shp in (("q", (Fd, L)), ("k", (Fd, L)), ("v", (Fd, L)), ("att", (Fd, L)), ("sm", (h, L, L))):
            names[n] = self._t("mhsa_" + n, shp)
        zb = self._t("mhsa_zero_bias", (Fd,))
        tmax = max(L * L, E * Fd, L * Fd, E * L)
        temp, grad, maxes, sums = self._t("mhsa_temp", (tmax,)), self._t("mhsa_grad", (L * L,)), self._t("mhsa_maxes", (L,)), self._t("mhsa_sums", (L,))
        b2 = lambda n, Hh, Ww: self.pkg.make_blob(self.keep, self.d(n), self.g(n), C=1, H=Hh, W=Ww, half=self.half)
        nodiff = lambda n, Hh, Ww: self.pkg.make_blob(self.keep, self.d(n), None, C=1, H=Hh, W=Ww, half=self.half)
        bias = lambda: self.pkg.make_blob(self.keep, self.d(zb), self.g(zb), dim=Fd, W=Fd, half=self.half)
        a = self.pkg.make_args(self.keep, "Mhsa_args" + self.sfx, input=b2(x, L, E), input_bn=nodiff(x, L, E), n_heads=h, output=b2(y, L, Fd),
                               coeff_in_q=b2("Wq", Fd, E), coeff_in_k=b2("Wk", Fd, E), coeff_in_v=b2("Wv", Fd, E), coeff_out=b2("Wo", Fd, Fd),
                               bias_in_q=bias(), bias_in_k=bias(), bias_in_v=bias(), bias_out=bias(),
                               q=b2(names["q"], L, Fd), k=b2(names["k"], L, Fd), v=b2(names["v"], L, Fd), attention_map=b2(names["att"], L, Fd),
                               temp_buffer=self.d(temp), grad=self.d(grad), softmax_buffer=b2(names["sm"], h, L * L), maxes=self.d(maxes), sums=self.d(sums),
                               opt_matmul_type_fw=0, opt_matmul_type_wg=0, opt_matmul_type_ig=0)
        t = "fp16" if self.half else "fp32"
        self._call(self.fw, "pulp_mhsa_mobilebert_inference_%s_fw_cl" % t, a)
        bw = []
        zero = self.pkg.make_args(self.keep, "transp_args" + self.sfx, in_matrix=self.d("zeros_EL"), out_matrix=self.g(x), N=1, M=E * L)
        self._call(bw, "transpose_matrix" + self.sfx, zero)                       # the backward accumulates into input.diff: clear it (copy of zeros)
        self._call(bw, "pulp_mhsa_mobilebert_inference_%s_bw_cl" % t, a)
        return bw

    # ---------------------------------------------------------------- graph of the block
    def setup_device(self):
        rng = np.random.default_rng(4)
        L, H, B, FF = self.L, self.H, self.B, self.FF
        rnd = lambda *s: np.float32(0.02) * rng.standard_normal(s).astype(F)
        P = lambda name, arr: (self._t(name, arr.shape, arr), self.params.append(name))[0]
        self.eps_host = np.array([1e-3], self.dt)          # read on the host by the layer-norm entry points
        self._t("zeros_EL", (B * L,))
        X = self._t("X", (L, H), rng.standard_normal((L, H)).astype(F))
        T = self._t("target", (L, H), rng.standard_normal((L, H)).astype(F))
        P("Wbi", rnd(H, B)); P("Wbo", rnd(B, H))
        for n in ("Wq", "Wk", "Wv", "Wo"):
            P(n, rnd(B, B))
        ln = lambda name, width: (P(name + "_w", 1 + rnd(width)), P(name + "_b", rnd(width)))
        # forward calls are appended to self.fw as the layers are declared; every layer hands back its backward calls, which are
        # put together below in reverse order (a residual's copy before its branch, its add after it)
        t0, x1 = self._t("t0", (L, B)), self._t("x1", (L, B))
        bw_lin_bi = self.linear(X, "Wbi", t0); w, b = ln("ln1", B); bw_ln1 = self.layernorm(t0, w, b, x1)
        att, r1, x = self._t("att", (L, B)), self._t("r1", (L, B)), self._t("x2", (L, B))
        bw_mhsa = self.mhsa(x1, att)
        res1_copy, res1_add = self.residual(x1, att, r1)
        w, b = ln("ln2", B); bw_ln2 = self.layernorm(r1, w, b, x)
        ffn_bw = []
        for f in range(self.NFFN):
            P("W1_%d" % f, rnd(B, FF)); P("W2_%d" % f, rnd(FF, B))
            h, gl, o, r, xn = [self._t("%s_%d" % (n, f), sh) for n, sh in (("h", (L, FF)), ("gelu", (L, FF)), ("o", (L, B)), ("r", (L, B)), ("xf", (L, B)))]
            b1 = self.linear(x, "W1_%d" % f, h); bg = self.gelu(h, gl); b2 = self.linear(gl, "W2_%d" % f, o)
            cp, ad = self.residual(x, o, r)
            w, b = ln("lnf_%d" % f, B); bl = self.layernorm(r, w, b, xn)
            ffn_bw.append(bl + cp + b2 + bg + b1 + ad)
            x = xn
        t1, r2, Y = self._t("t1", (L, H)), self._t("r2", (L, H)), self._t("Y", (L, H))
        bw_lin_bo = self.linear(x, "Wbo", t1)
        reso_copy, reso_add = self.residual(X, t1, r2)
        w, b = ln("ln_out", H); bw_ln_out = self.layernorm(r2, w, b, Y)
        self._t("loss", (1,))
        la = self.pkg.make_args(self.keep, "loss_args" + self.sfx, output=self._blob(Y), target=self.d(T), wr_loss=self.d("loss"))
        self._call(self.fw, "pulp_MSELoss" + self.sfx, la)
        bw_loss = []
        self._call(bw_loss, "pulp_MSELoss_backward" + self.sfx, la)
        # loss scaling, as fp16 training does: dL/dY = 2 (y - t) / 65536 is about 3e-5, inside the fp16 subnormal range, and the
        # attention gradients behind it would underflow; every gradient below is LOSS_SCALE times the true one
        n_y = int(np.prod(self.shape(Y)))
        sa = self.pkg.make_args(self.keep, "scalar_mul_args" + self.sfx, input=self.g(Y), scalar=self.LOSS_SCALE, dim=n_y)
        self._call(bw_loss, "pulp_scalar_mul_%s_cl" % ("fp16" if self.half else "fp32"), sa)
        flat = bw_loss + bw_ln_out + reso_copy + bw_lin_bo
        for piece in reversed(ffn_bw):
            flat += piece
        flat += bw_ln2 + res1_copy + bw_mhsa + res1_add + bw_ln1 + bw_lin_bi + reso_add
        self.bw_flat = flat
        self.flush = self.pkg.DeviceBuffer(self.lib, nbytes=256 << 20)

    def step_device(self):
        for fn, a in self.fw:
            fn(ctypes.byref(a))
        for fn, a in self.bw_flat:
            fn(ctypes.byref(a))

    # the block has no host-pointer form here: its end-to-end number uploads the input and target and reads back the loss
    def setup_host(self, lib):
        if not hasattr(lib, "trainlib_malloc_host"):
            raise SystemExit("config 4 has no reference arm: " + self.no_reference)
        from bench import pinned_like
        self.hX = pinned_like(self.pkg, lib, self.get("X").astype(self.dt)); self.hT = pinned_like(self.pkg, lib, self.get("target").astype(self.dt))
        self.hloss = pinned_like(self.pkg, lib, np.zeros(1, self.dt))
        self.h2d = self.hX.nbytes + self.hT.nbytes; self.d2h = self.hloss.nbytes

    def step_host(self, lib):
        lib.trainlib_memcpy_h2d(self.d("X"), self.hX.ctypes.data, self.hX.nbytes)
        lib.trainlib_memcpy_h2d(self.d("target"), self.hT.ctypes.data, self.hT.nbytes)
        self.step_device()
        lib.trainlib_memcpy_d2h(self.hloss.ctypes.data, self.d("loss"), self.hloss.nbytes)

    def metric(self, ms):
        return {"metric": "fw_bw_tflops", "unit": "TFLOP/s", "value": self.flops / (ms * 1e-3) / 1e12}

    def roofline(self, ms, pk):
        tf = self.flops / (ms * 1e-3) / 1e12
        peak = pk["bf16_tflops_sustained"] if self.half else pk["bf16_tflops_sustained"] / 6.0
        return {"bound": "tensor", "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak, "traffic": None, "peak_source": pk["source"],
                "kernel": "whole block: %d forward + %d backward entry-point calls" % (len(self.fw), len(self.bw_flat)), "algorithmic_flops": self.flops,
                "us_per_step": 1e3 * ms, "peak_note": "products of 128 x 128..512 x 128..512: launch-latency bound, far below any roofline"}
