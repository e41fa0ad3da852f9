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
                "kernel": "attention forward + backward (strided / batched FFMA GEMMs + softmax kernels)", "algorithmic_flops": self.flops,
                "algorithmic_bytes": self.bytes, "us_per_step": 1e3 * ms,
                "peak_note": "FFMA peak measured on this part (125 MAC/clk/SM); the 256^3 products stay on the FFMA tiles because their summation "
                             "order keeps the backward inside 1e-5 of the reference"}
