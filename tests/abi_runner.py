"""Drives any library that exports the PULP-TrainLib C ABI - the reference compiled for the host
(oracle/_ref/libpulp_ref.so) or libtrainlib_b200.so - through the same argument structs.

`device=True` (only meaningful for libtrainlib_b200) keeps every tensor in device memory and
passes device pointers; otherwise the structs point at numpy arrays on the host.
"""
import ctypes

import numpy as np


class Tens(object):
    """One tensor handed to the library: host numpy array or device buffer."""

    def __init__(self, runner, array):
        self.r = runner
        self.host = np.array(array, order="C", copy=True)     # the library may write through it
        self.dev = None
        if runner.device:
            self.dev = runner.pkg.DeviceBuffer(runner.lib, self.host)

    @property
    def arg(self):
        return self.dev.ptr if self.dev is not None else self.host

    def get(self):
        if self.dev is not None:
            return self.dev.download(self.host.dtype, self.host.shape)
        return self.host

    def set(self, array):
        """overwrite the tensor in place (same address: recorded graphs keep pointing at it)"""
        self.host[...] = np.asarray(array, dtype=self.host.dtype).reshape(self.host.shape)
        if self.dev is not None:
            self.dev.upload(self.host)

    def free(self):
        if self.dev is not None:
            self.dev.free()
            self.dev = None


class AbiRunner(object):
    def __init__(self, pkg, lib, device=False, half=False, is_ref=False):
        self.pkg, self.lib, self.device, self.half, self.is_ref = pkg, lib, device, half, is_ref
        self.dt = np.float16 if half else np.float32
        self.sfx = "_fp16" if half else ""
        self.keep = pkg.Keep()
        self.tensors = []

    # ---------------------------------------------------------------- plumbing
    def t(self, array):
        x = Tens(self, np.asarray(array, dtype=self.dt))
        self.tensors.append(x)
        return x

    def zeros(self, *shape):
        return self.t(np.zeros(shape, self.dt))

    def blob(self, data=None, diff=None, C=1, H=1, W=1, dim=None):
        return self.pkg.make_blob(self.keep, data.arg if data is not None else None, diff.arg if diff is not None else None,
                                  C=C, H=H, W=W, dim=dim, half=self.half)

    def args(self, name, **fields):
        conv = {k: (v.arg if isinstance(v, Tens) else v) for k, v in fields.items()}
        return self.pkg.make_args(self.keep, name, **conv)

    def call(self, fn, args):
        getattr(self.lib, fn)(ctypes.byref(args))
        if not self.is_ref:
            self.pkg.check(self.lib)

    def close(self):
        for x in self.tensors:
            x.free()
        self.tensors = []

    def sname(self, base):
        """struct name of the fp32/fp16 family"""
        special = {"array_broadcast_sum_args": ("array_broadcast_sum_fp32_args", "array_broadcast_sum_fp16_args")}
        if base in special:
            return special[base][1 if self.half else 0]
        return base + self.sfx

    def fname(self, base32):
        """function name: fp32 names carry 'fp32' where the fp16 twin carries 'fp16'"""
        if not self.half:
            return base32
        if "fp32" in base32:
            return base32.replace("fp32", "fp16")
        return base32 + "_fp16"

    # ---------------------------------------------------------------- primitives
    def mm(self, A, B, N, K, M, trans_B=0, fn="mm", C0=None):
        a, b = self.t(A), self.t(B)
        c = self.t(C0) if C0 is not None else self.zeros(N, M)
        args = self.args(self.sname("matMul_args"), A=a, B=b, C=c, N=N, K=K, M=M, trans_B=trans_B, USE_BIASES=0)
        self.call(fn if not self.half else (fn + "_fp16" if "fp16" not in fn else fn), args)
        return c.get()

    def conv2d(self, x, w, dy, g, use_im2col=0, bias=None, steps=("fw", "wg", "ig"), hwc=0):
        """hwc=1: x, dy and the results are [H][W][C], w is [Cout][Hk][Wk][Cin] (only the flat sizes matter to the structs)"""
        from oracle_bind import out_hw
        Ho, Wo = out_hw(g)
        X, W_ = self.t(x), self.t(w)
        Y, dX, dW, dY = self.zeros(g["Cout"], Ho, Wo), self.zeros(*x.shape), self.zeros(*w.shape), self.t(dy if dy is not None else np.zeros((g["Cout"], Ho, Wo)))
        B = self.t(bias if bias is not None else np.zeros(g["Cout"]))
        dB = self.zeros(g["Cout"])
        K = g["Cin"] * g["Hk"] * g["Wk"]
        # scratch sized as the reference's im2col path needs it
        i2c = self.zeros(max(Ho * Wo * K, g["Hin"] * g["Win"] * g["Cout"] * g["Hk"] * g["Wk"]) if (self.is_ref and use_im2col) else 1)
        bt = self.zeros(w.size if (self.is_ref and use_im2col) else 1)
        bin_ = self.blob(X, dX, C=g["Cin"], H=g["Hin"], W=g["Win"])
        bw = self.blob(W_, dW, C=g["Cin"], H=g["Hk"], W=g["Wk"], dim=w.size)
        bb = self.blob(B, dB, C=1, H=1, W=g["Cout"], dim=g["Cout"])
        bout = self.blob(Y, dY, C=g["Cout"], H=Ho, W=Wo)
        args = self.args(self.sname("Conv2D_args"), input=bin_, coeff=bw, bias=bb, output=bout,
                         Lpad=g["padL"], Rpad=g["padR"], Upad=g["padU"], Dpad=g["padD"], stride_h=g["sh"], stride_w=g["sw"],
                         i2c_buffer=i2c, bt_buffer=bt, skip_wg_grad=0, skip_in_grad=0, HWC=hwc,
                         opt_matmul_type_fw=0, opt_matmul_type_wg=0, opt_matmul_type_ig=0,
                         USE_BIASES=1 if bias is not None else 0, USE_IM2COL=use_im2col, USE_DMA_IM2COL=0)
        r = {}
        if "fw" in steps:
            self.call(self.fname("pulp_conv2d_fp32_fw_cl"), args); r["y"] = Y.get().copy()
        if "wg" in steps:
            self.call(self.fname("pulp_conv2d_fp32_bw_param_grads_cl"), args); r["dw"] = dW.get().copy(); r["db"] = dB.get().copy()
        if "ig" in steps:
            self.call(self.fname("pulp_conv2d_fp32_bw_input_grads_cl"), args); r["dx"] = dX.get().copy()
        return r

    def pw(self, x, w, dy, Cin, Cout, H, W, hwc=0):
        X, W_, dY = self.t(x), self.t(w), self.t(dy)
        Y, dX, dW, tr = self.zeros(*dy.shape), self.zeros(*x.shape), self.zeros(*w.shape), self.zeros(max(w.size, x.size))
        args = self.args(self.sname("PointWise_Conv_args"), input=self.blob(X, dX, C=Cin, H=H, W=W),
                         coeff=self.blob(W_, dW, C=Cin, H=1, W=1, dim=w.size), output=self.blob(Y, dY, C=Cout, H=H, W=W),
                         transpose_buffer=tr, skip_wg_grad=0, skip_in_grad=0, opt_matmul_type_fw=0, opt_matmul_type_wg=0,
                         opt_matmul_type_ig=0, HWC=hwc)
        self.call(self.fname("pulp_conv_pw_fp32_fw_cl"), args)
        self.call(self.fname("pulp_conv_pw_fp32_bw_cl"), args)
        return dict(y=Y.get().copy(), dw=dW.get().copy(), dx=dX.get().copy())

    def dw(self, x, w, dy, g):
        from oracle_bind import out_hw
        Ho, Wo = out_hw(g)
        X, W_, dY = self.t(x), self.t(w), self.t(dy)
        Y, dX, dW = self.zeros(g["Cin"], Ho, Wo), self.zeros(*x.shape), self.zeros(*w.shape)
        fields = dict(input=self.blob(X, dX, C=g["Cin"], H=g["Hin"], W=g["Win"]), coeff=self.blob(W_, dW, C=g["Cin"], H=g["Hk"], W=g["Wk"]),
                      output=self.blob(Y, dY, C=g["Cin"], H=Ho, W=Wo), Lpad=g["padL"], Rpad=g["padR"], Upad=g["padU"], Dpad=g["padD"],
                      skip_wg_grad=0, skip_in_grad=0, HWC=0)
        if not self.half:
            fields.update(stride_h=g["sh"], stride_w=g["sw"])
        args = self.args(self.sname("DepthWise_Conv_args"), **fields)
        self.call(self.fname("pulp_conv_dw_fp32_fw_cl"), args)
        self.call(self.fname("pulp_conv_dw_fp32_bw_cl"), args)
        return dict(y=Y.get().copy(), dw=dW.get().copy(), dx=dX.get().copy())

    def linear(self, Wm, x, dy, bias=None, n=1, one_backward_call=False):
        out, inn = Wm.shape
        W_, X, dY = self.t(Wm), self.t(x), self.t(dy)
        Y, dW, dX = self.zeros(n * out), self.zeros(out, inn), self.zeros(n * inn)
        B, dB = self.t(bias if bias is not None else np.zeros(out)), self.zeros(out)
        args = self.args(self.sname("Linear_args"), input=self.blob(X, dX, C=1, H=1, W=inn, dim=inn),
                         coeff=self.blob(W_, dW, C=1, H=out, W=inn, dim=out * inn), bias=self.blob(B, dB, dim=out, W=out),
                         output=self.blob(Y, dY, C=1, H=1, W=out, dim=out), skip_wg_grad=0, skip_in_grad=0,
                         opt_matmul_type_fw=0, opt_matmul_type_wg=0, opt_matmul_type_ig=0, use_biases=1 if bias is not None else 0)
        self.call(self.fname("pulp_linear_fp32_fw_cl"), args)
        if one_backward_call:
            self.call(self.fname("pulp_linear_fp32_bw_cl"), args)
        else:
            self.call(self.fname("pulp_linear_fp32_bw_param_grads_cl"), args)
            self.call(self.fname("pulp_linear_fp32_bw_input_grads_cl"), args)
        return dict(y=Y.get().copy(), dW=dW.get().copy(), dx=dX.get().copy(), db=dB.get().copy())

    def mhsa(self, x, wq, wk, wv, bq, bk, bv, wo, dy, L, E, F, heads):
        z = self.zeros
        X, dX = self.t(x), z(E, L)
        ws = [self.t(a) for a in (wq, wk, wv, wo)]
        dws = [z(F, E), z(F, E), z(F, E), z(E, F)]
        bs = [self.t(a) for a in (bq, bk, bv)]
        dbs = [z(F), z(F), z(F)]
        q, k, v, att = z(F, L), z(F, L), z(F, L), z(F, L)
        dq, dk, dv, datt = z(F, L), z(F, L), z(F, L), z(F, L)
        sm, dsm = z(heads, L, L), z(heads, L, L)
        Y, dY = z(E, L), self.t(dy if dy is not None else np.zeros((E, L)))
        tmax = max(L * L, E * F, L * F, E * L)
        temp, grad, maxes, sums = z(tmax), z(L * L), z(L), z(L)
        args = self.args(self.sname("Mhsa_args"),
                         input=self.blob(X, dX, C=1, H=L, W=E), n_heads=heads, output=self.blob(Y, dY, C=1, H=L, W=E),
                         coeff_in_q=self.blob(ws[0], dws[0], C=1, H=F, W=E), coeff_in_k=self.blob(ws[1], dws[1], C=1, H=F, W=E),
                         coeff_in_v=self.blob(ws[2], dws[2], C=1, H=F, W=E), coeff_out=self.blob(ws[3], dws[3], C=1, H=E, W=F),
                         bias_in_q=self.blob(bs[0], dbs[0], dim=F, W=F), bias_in_k=self.blob(bs[1], dbs[1], dim=F, W=F),
                         bias_in_v=self.blob(bs[2], dbs[2], dim=F, W=F),
                         q=self.blob(q, dq, C=1, H=L, W=F), k=self.blob(k, dk, C=1, H=L, W=F), v=self.blob(v, dv, C=1, H=L, W=F),
                         attention_map=self.blob(att, datt, C=1, H=L, W=F), temp_buffer=temp, grad=grad,
                         softmax_buffer=self.blob(sm, dsm, C=1, H=heads, W=L * L), maxes=maxes, sums=sums,
                         opt_matmul_type_fw=0, opt_matmul_type_wg=0, opt_matmul_type_ig=0)
        self.call(self.fname("pulp_mhsa_fp32_fw_cl"), args)
        r = dict(y=Y.get().copy(), q=q.get().copy(), k=k.get().copy(), v=v.get().copy(), softmax=sm.get().copy(), att=att.get().copy())
        if dy is not None:
            self.call(self.fname("pulp_mhsa_fp32_bw_cl"), args)
            r.update(dx=dX.get().copy(), dwq=dws[0].get().copy(), dwk=dws[1].get().copy(), dwv=dws[2].get().copy(), dwo=dws[3].get().copy(),
                     dq=dq.get().copy(), dk=dk.get().copy(), dv=dv.get().copy(), datt=datt.get().copy(), dsoftmax=dsm.get().copy())
        return r

    def mobilebert(self, x, xb, wq, wk, wv, bq, bk, bv, wo, bo, dy, L, E, Kb, F, No, heads, tiled=False, share_input_diff=False):
        """MobileBERT attention: x L x E, xb L x Kb, Wq/Wk F x Kb, Wv F x E, Wo No x F, output L x No.  `tiled` calls
        tiled_mhsa_* (sizes from the coefficient blobs) instead of the inference entry point (F = Kb = No);
        dy = None skips the backward (the reference library has none that compiles)."""
        z = self.zeros
        X, dX, XB, dXB = self.t(x), z(L, E), self.t(xb), z(L, Kb)
        ws = [self.t(a) for a in (wq, wk, wv, wo)]
        dws = [z(F, Kb), z(F, Kb), z(F, E), z(No, F)]
        bs = [self.t(a) for a in (bq, bk, bv, bo)]
        dbs = [z(F), z(F), z(F), z(No)]
        q, k, v, att = z(F, L), z(F, L), z(F, L), z(F, L)
        dq, dk, dv, datt = z(F, L), z(F, L), z(F, L), z(F, L)
        sm, dsm = z(heads, L, L), z(heads, L, L)
        Y, dY = z(L, No), self.t(dy if dy is not None else np.zeros((L, No)))
        tmax = max(L * L, F * Kb, L * F, E * L, No * L, F * E)
        temp, grad, maxes, sums = z(tmax), z(L * L), z(L), z(L)
        args = self.args(self.sname("Mhsa_args"),
                         input=self.blob(X, dX, C=1, H=L, W=E), input_bn=self.blob(XB, None if share_input_diff else dXB, C=1, H=L, W=Kb),
                         n_heads=heads, output=self.blob(Y, dY, C=1, H=L, W=No),
                         coeff_in_q=self.blob(ws[0], dws[0], C=1, H=F, W=Kb), coeff_in_k=self.blob(ws[1], dws[1], C=1, H=F, W=Kb),
                         coeff_in_v=self.blob(ws[2], dws[2], C=1, H=F, W=E), coeff_out=self.blob(ws[3], dws[3], C=1, H=No, W=F),
                         bias_in_q=self.blob(bs[0], dbs[0], dim=F, W=F), bias_in_k=self.blob(bs[1], dbs[1], dim=F, W=F),
                         bias_in_v=self.blob(bs[2], dbs[2], dim=F, W=F), bias_out=self.blob(bs[3], dbs[3], dim=No, W=No),
                         q=self.blob(q, dq, C=1, H=L, W=F), k=self.blob(k, dk, C=1, H=L, W=F), v=self.blob(v, dv, C=1, H=L, W=F),
                         attention_map=self.blob(att, datt, C=1, H=L, W=F), temp_buffer=temp, grad=grad,
                         softmax_buffer=self.blob(sm, dsm, C=1, H=heads, W=L * L), maxes=maxes, sums=sums,
                         opt_matmul_type_fw=0, opt_matmul_type_wg=0, opt_matmul_type_ig=0)
        if tiled:
            targs = self.args(self.sname("Tiled_Matmul_Mhsa_args"), tile_h=1, tile_w=1, tile_dim=1)
            getattr(self.lib, "tiled_mhsa_fp16" if self.half else "tiled_mhsa_fp32")(ctypes.byref(args), ctypes.byref(targs))
            self.pkg.check(self.lib)
        else:
            self.call(self.fname("pulp_mhsa_mobilebert_inference_fp32_fw_cl"), args)
        r = dict(y=Y.get().copy(), q=q.get().copy(), k=k.get().copy(), v=v.get().copy(), softmax=sm.get().copy(), att=att.get().copy())
        if dy is not None:
            self.call(self.fname("pulp_mhsa_mobilebert_inference_fp32_bw_cl"), args)
            r.update(dx=dX.get().copy(), dxb=dXB.get().copy(), dwq=dws[0].get().copy(), dwk=dws[1].get().copy(), dwv=dws[2].get().copy(),
                     dwo=dws[3].get().copy(), dq=dq.get().copy(), dk=dk.get().copy(), dv=dv.get().copy(), datt=datt.get().copy(),
                     dsoftmax=dsm.get().copy())
        return r

    def act(self, kind, x, dy, slope=0.01):
        """kind: relu | leakyrelu | sigmoid | gelu"""
        X, dX, Y, dY = self.t(x), self.zeros(*x.shape), self.zeros(*x.shape), self.t(dy)
        bi, bo = self.blob(X, dX, dim=x.size, W=x.size), self.blob(Y, dY, dim=x.size, W=x.size)
        if kind == "leakyrelu":
            args = self.args(self.sname("leakyrelu_args"), input=bi, output=bo, negative_slope=slope)
        else:
            args = self.args(self.sname("act_args"), input=bi, output=bo, H=1, W=x.size)
        if kind == "gelu":
            self.call("pulp_gelu_fp16_fw_cl" if self.half else "pulp_gelu_tanh_approx_fp32_fw_cl", args)
            return dict(y=Y.get().copy())
        self.call(self.fname("pulp_%s_fp32_fw_cl" % kind), args)
        y = Y.get().copy()
        self.call(self.fname("pulp_%s_fp32_bw_cl" % kind), args)
        return dict(y=y, dx=dX.get().copy())

    def softmax(self, x, dout):
        H, W = x.shape
        X, OUT, dOUT, dIN = self.t(x), self.zeros(H, W), self.t(dout), self.zeros(H, W)
        mx, sm = self.zeros(H), self.zeros(H)
        args = self.args(self.sname("softmax_args"), input_data=X, input_diff=dIN, output_data=OUT, output_diff=dOUT,
                         H=H, W=W, L=W, n_heads=1, maxes=mx, sums=sm)
        self.call(self.fname("pulp_softmax_fp32_fw_cl"), args)
        out = OUT.get().copy()
        self.call(self.fname("pulp_softmax_fp32_bw_cl"), args)
        return dict(out=out, din=dIN.get().copy())

    def instnorm(self, x, gb, dy):
        C, H, W = x.shape
        X, dX, Y, dY = self.t(x), self.zeros(C, H, W), self.zeros(C, H, W), self.t(dy)
        GB, dGB = self.t(gb), self.zeros(2 * C)
        m, v, s = self.zeros(C), self.zeros(C), self.zeros(C)
        args = self.args(self.sname("InstNorm_args"), input=self.blob(X, dX, C=C, H=H, W=W), output=self.blob(Y, dY, C=C, H=H, W=W),
                         coeff=self.blob(GB, dGB, dim=2 * C, W=2 * C), running_mean=m, running_var=v, running_stdev=s,
                         freeze_running_params=0, skip_wg_grad=0, skip_in_grad=0)
        self.call(self.fname("pulp_instnorm_fp32_fw_cl"), args)
        y = Y.get().copy()
        self.call(self.fname("pulp_instnorm_fp32_bw_cl"), args)
        return dict(y=y, dx=dX.get().copy(), dgb=dGB.get().copy(), mean=m.get().copy(), var=v.get().copy(), std=s.get().copy())

    def batchnorm_fw(self, x, w, b, B, C, H, W, eps):
        X, Y, Wt, Bt = self.t(x), self.zeros(*x.shape), self.t(w), self.t(b)
        epsv = np.array([eps], np.float32)
        args = self.args("BatchNorm_args_fp32", input=self.blob(X, None, C=C, H=H, W=W, dim=x.size), output=self.blob(Y, None, C=C, H=H, W=W, dim=x.size),
                         weight_data=Wt, bias_data=Bt, eps=self.keep.hold(epsv), B=B, C=C, H=H, W=W, batch_size=B)
        self.call("pulp_batch_norm_fp32_fw_cl", args)
        return Y.get().copy()

    def layernorm_fw(self, x, w, b, rows, width, eps):
        X, Y, Wt, Bt = self.t(x), self.zeros(*x.shape), self.t(w), self.t(b)
        epsv = np.array([eps], np.float32)
        args = self.args("LayerNorm_args_fp32", x=X, weight=Wt, bias=Bt, output=Y, eps=self.keep.hold(epsv), size=rows * width, step_size=width)
        self.call("pulp_layerNorm_fp32_fw_cl", args)     # the reference worker runs as core 0 of 1
        return Y.get().copy()

    def mm_broadcast(self, A, B):
        a, b = self.t(A), self.t(B)
        out_shape = np.broadcast_shapes(A.shape[:-2], B.shape[:-2]) + (A.shape[-2], B.shape[-1])
        c = self.zeros(*out_shape)
        ad = (ctypes.c_int * A.ndim)(*A.shape); bd = (ctypes.c_int * B.ndim)(*B.shape)
        args = self.args("broadcastMatMul_args_fp16" if self.half else "broadcastMatMul_args_fp32", A=a, B=b, C=c,
                         A_dims=self.keep.hold(ad), B_dims=self.keep.hold(bd), A_dims_len=A.ndim, B_dims_len=B.ndim)
        self.call("mm_broadcast_fp16" if self.half else "mm_broadcast_fp32", args)
        return c.get().reshape(out_shape)

    def layernorm_ext(self, x, w, b, dy, rows, width, eps):
        """layer norm through the library's own struct (fp16 forward and both backward passes are not in the reference)"""
        import ctypes

        class LnArgs(ctypes.Structure):
            _fields_ = [(n, ctypes.c_void_p) for n in ("x", "weight", "bias", "output", "eps")] + [("size", ctypes.c_int), ("step_size", ctypes.c_int)] + \
                       [(n, ctypes.c_void_p) for n in ("dy", "dx", "dweight", "dbias")]
        X, Y, Wt, Bt, dY = self.t(x), self.zeros(*x.shape), self.t(w), self.t(b), self.t(dy)
        dX, dW, dB, E = self.zeros(*x.shape), self.zeros(width), self.zeros(width), self.t(np.array([eps]))
        a = LnArgs()
        for n, t in (("x", X), ("weight", Wt), ("bias", Bt), ("output", Y), ("eps", E), ("dy", dY), ("dx", dX), ("dweight", dW), ("dbias", dB)):
            setattr(a, n, t.arg if isinstance(t.arg, int) else t.arg.ctypes.data)
        a.size, a.step_size = rows * width, width
        self.keep.hold(a)
        getattr(self.lib, "trainlib_layernorm_fp16_fw_cl" if self.half else "pulp_layerNorm_fp32_fw_cl")(ctypes.byref(a))
        getattr(self.lib, "trainlib_layernorm_fp16_bw_cl" if self.half else "trainlib_layernorm_fp32_bw_cl")(ctypes.byref(a))
        self.pkg.check(self.lib)
        return dict(y=Y.get().copy(), dx=dX.get().copy(), dw=dW.get().copy(), db=dB.get().copy())

    def instnorm_act(self, x, gb, dy, skip=None, relu=True, backward=True, n=1, diff2=None):
        """the library's fused norm (+ skip sum) (+ ReLU): one forward call, one backward call; x is [n][C][H][W] when n > 1"""
        import ctypes

        class FusedArgs(ctypes.Structure):
            _fields_ = [("norm", ctypes.c_void_p), ("skip", ctypes.c_void_p), ("relu", ctypes.c_int), ("diff2", ctypes.c_void_p)]
        C, H, W = x.shape[-3:]
        X, dX, Y, dY = self.t(x), self.zeros(*x.shape), self.zeros(*x.shape), self.t(dy)
        GB, dGB = self.t(gb), self.zeros(2 * C)
        m, v, s = self.zeros(n * C), self.zeros(n * C), self.zeros(n * C)
        norm = self.args(self.sname("InstNorm_args"), input=self.blob(X, dX, C=C, H=H, W=W), output=self.blob(Y, dY, C=C, H=H, W=W),
                         coeff=self.blob(GB, dGB, dim=2 * C, W=2 * C), running_mean=m, running_var=v, running_stdev=s,
                         freeze_running_params=0, skip_wg_grad=0, skip_in_grad=0)
        f = FusedArgs(); f.norm = ctypes.addressof(norm); f.relu = 1 if relu else 0
        if skip is not None:
            S = self.t(skip); sb = self.blob(S, None, C=C, H=H, W=W); f.skip = ctypes.addressof(sb)
        if diff2 is not None:
            D2 = self.t(diff2); f.diff2 = D2.arg if isinstance(D2.arg, int) else D2.arg.ctypes.data
        self.keep.hold(f)
        getattr(self.lib, self.fname("trainlib_instnorm_act_fp32_fw_cl"))(ctypes.byref(f)); self.pkg.check(self.lib)
        out = dict(y=Y.get().copy(), mean=m.get().copy(), std=s.get().copy())
        if backward:
            getattr(self.lib, self.fname("trainlib_instnorm_act_fp32_bw_cl"))(ctypes.byref(f)); self.pkg.check(self.lib)
            out.update(dx=dX.get().copy(), dgb=dGB.get().copy())
        return out

    def gelu_bw(self, x, dy):
        import ctypes
        X, dX, Y, dY = self.t(x), self.zeros(*x.shape), self.zeros(*x.shape), self.t(dy)
        args = self.args(self.sname("act_args"), input=self.blob(X, dX, dim=x.size, W=x.size), output=self.blob(Y, dY, dim=x.size, W=x.size), H=1, W=x.size)
        getattr(self.lib, "trainlib_gelu_fp16_bw_cl" if self.half else "trainlib_gelu_fp32_bw_cl")(ctypes.byref(args))
        self.pkg.check(self.lib)
        return dX.get().copy()

    def loss(self, kind, y, t):
        """kind: MSELoss | CrossEntropyLoss"""
        Y, dY, T = self.t(y), self.zeros(*y.shape), self.t(t)
        L = self.zeros(1)
        args = self.args(self.sname("loss_args"), output=self.blob(Y, dY, dim=y.size, W=y.size), target=T, wr_loss=L)
        f, b = "pulp_%s" % kind, "pulp_%s_backward" % kind
        self.call(f + self.sfx, args)
        loss = L.get().copy()[0]
        self.call(b + self.sfx, args)
        return loss, dY.get().copy()

    def sgd(self, w, g, lr, lam=0.0, bias=None, bias_g=None):
        W_, G = self.t(w), self.t(g)
        fields = dict(weights=self.blob(W_, G, dim=w.size, W=w.size), learning_rate=lr, weight_decay_lambda=lam, use_biases=0)
        if bias is not None:
            Bt, BG = self.t(bias), self.t(bias_g)
            fields.update(biases=self.blob(Bt, BG, dim=bias.size, W=bias.size), use_biases=1)
        args = self.args(self.sname("optim_args"), **fields)
        self.call(self.fname("pulp_gradient_descent_fp32"), args)
        r = dict(w=W_.get().copy(), g=G.get().copy())
        if bias is not None:
            r.update(b=Bt.get().copy())
        return r

    def residual(self, skip, lout, dout, dskip0):
        S, dS, Lo, dLo = self.t(skip), self.t(dskip0), self.t(lout), self.zeros(*lout.shape)
        O, dO = self.zeros(*skip.shape), self.t(dout)
        n = skip.size
        args = self.args(self.sname("SkipConn_args"), skip=self.blob(S, dS, dim=n, W=n), lout=self.blob(Lo, dLo, dim=n, W=n),
                         output=self.blob(O, dO, dim=n, W=n), skip_in_grad=0)
        self.call(self.fname("pulp_residualconn_fp32_fw"), args)
        self.call(self.fname("pulp_sumnode_fp32_bw"), args)
        self.call(self.fname("pulp_residualconn_fp32_bw"), args)
        return dict(out=O.get().copy(), dskip=dS.get().copy(), dlout=dLo.get().copy())

    def avgpool(self, x, dy, Hk, Wk, sh, sw):
        C, H, W = x.shape
        Ho, Wo = (H - Hk + sh) // sh, (W - Wk + sw) // sw
        X, dX, Y, dY = self.t(x), self.zeros(C, H, W), self.zeros(C, Ho, Wo), self.t(dy)
        args = self.args(self.sname("pool_args"), input=self.blob(X, dX, C=C, H=H, W=W), output=self.blob(Y, dY, C=C, H=Ho, W=Wo),
                         Hker=Hk, Wker=Wk, Hstride=sh, Wstride=sw)
        self.call(self.fname("pulp_avgpool_fp32_fw_cl"), args)
        self.call(self.fname("pulp_avgpool_fp32_bw_cl"), args)
        return dict(y=Y.get().copy(), dx=dX.get().copy())

    def family(self, i):
        """The rest of the element-wise family on the inputs of golden_cases._Family; returns every output by name."""
        r = {}
        h = self.half
        nm = lambda base: base + ("_fp16" if h else "")            # names that append _fp16
        # --- L1 and berHu
        y, t = i["y"], i["t"]
        Y, dY, T, L = self.t(y), self.zeros(*y.shape), self.t(t), self.zeros(1)
        la = self.args(self.sname("loss_args"), output=self.blob(Y, dY, dim=y.size, W=y.size), target=T, wr_loss=L)
        self.call(nm("pulp_L1Loss"), la); r["l1"] = L.get().copy()
        self.call("pulp_L1Loss_backward" + self.sfx, la); r["l1_dy"] = dY.get().copy()
        ba = self.args(self.sname("berHu_loss_args"), output=self.blob(Y, dY, dim=y.size, W=y.size), target=T, wr_loss=L, alpha=float(i["alpha"][0]))
        self.call(nm("pulp_berHuLoss"), ba); r["berhu"] = L.get().copy()
        self.call("pulp_berHuLoss_backward" + self.sfx, ba); r["berhu_dy"] = dY.get().copy()
        # --- max pooling: disjoint 2x2 windows, and overlapping 3x3 stride-1 windows with ties
        for tag, x, g, (Hk, Wk, sh, sw) in (("mp2", i["px"], i["pdy2"], (2, 2, 2, 2)), ("mp3", i["pxt"], i["pdy3"], (3, 3, 1, 1))):
            C, H, W = x.shape
            Ho, Wo = (H - Hk + sh) // sh, (W - Wk + sw) // sw
            X, dX, O, dO = self.t(x), self.zeros(C, H, W), self.zeros(C, Ho, Wo), self.t(g)
            pa = self.args(self.sname("pool_args"), input=self.blob(X, dX, C=C, H=H, W=W), output=self.blob(O, dO, C=C, H=Ho, W=Wo), Hker=Hk, Wker=Wk, Hstride=sh, Wstride=sw)
            self.call(self.fname("pulp_maxpool_fp32_fw_cl"), pa); self.call(self.fname("pulp_maxpool_fp32_bw_cl"), pa)
            r[tag + "_y"] = O.get().copy(); r[tag + "_dx"] = dX.get().copy()
        # --- NoNorm
        nx = i["nx"]; rows, width = nx.shape
        NX, NW, NB, NO = self.t(nx), self.t(i["nw"]), self.t(i["nb"]), self.zeros(rows, width)
        na = self.args(self.sname("Nonorm_args"), input=self.blob(NX, None, C=1, H=rows, W=width), coeff=self.blob(NW, None, dim=width, W=width),
                       bias=self.blob(NB, None, dim=width, W=width), output=self.blob(NO, None, C=1, H=rows, W=width))
        self.call(self.fname("pulp_nonorm_fp32_fw_cl"), na); r["nonorm"] = NO.get().copy()
        # --- RMS norm and its pieces
        v, w = i["v"], i["w"]; n = v.size
        V, W_, O, B = self.t(v), self.t(w), self.zeros(n), self.zeros(8)
        wa = self.args(self.sname("weighted_scaling_args"), out=O, **{"in": V}, w=W_, scaling_factor=0.37, size=n)
        self.call(self.fname("weighted_scaling_fp32_cl"), wa); r["wscale"] = O.get().copy()
        sa = self.args(self.sname("sum_of_squares_args"), out=B, **{"in": V}, size=n)
        self.call(self.fname("sum_of_squares_fp32_cl"), sa); r["sumsq"] = B.get()[:1].copy()
        fn = getattr(self.lib, "rmsnorm_parallelized_fp16" if h else "rmsnorm_parallelized_fp32")
        fn.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int]; fn.restype = None
        ptr = lambda a: a.arg if not isinstance(a.arg, np.ndarray) else a.arg.ctypes.data
        fn(ptr(O), ptr(V), ptr(W_), ptr(B), n)
        if not self.is_ref:
            self.pkg.check(self.lib)
        r["rmsnorm"] = O.get().copy()
        # --- SwiGLU, vector softmax
        G1, G2, GO = self.t(v), self.t(w), self.zeros(n)
        ga = self.args(self.sname("swiglu_args"), in1=G1, in2=G2, out=GO, dim=n)
        self.call(self.fname("pulp_swiglu_fp32_cl"), ga); r["swiglu"] = GO.get().copy()
        fn = getattr(self.lib, "pulp_vector_softmax_fp16" if h else "pulp_vector_softmax_fp32")
        fn.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_uint]; fn.restype = None
        fn(ptr(GO), ptr(V), ptr(B), n)
        if not self.is_ref:
            self.pkg.check(self.lib)
        r["vsoftmax"] = GO.get().copy()
        # --- pieces of the softmax
        MX = self.zeros(8)
        ma = self.args(self.sname("max_args"), input=V, H=1, W=n, maxes=MX)
        self.call(self.fname("pulp_max_fp32_cl"), ma); r["vmax"] = MX.get()[:1].copy()
        EO, ES = self.zeros(n), self.zeros(8)
        ea = self.args(self.sname("vector_exp_sum_args"), input=V, sums=ES, output=EO, dim=n, max=float(v.max()))
        self.call("vector_exp_sum_fp16_cl" if h else "vector_exp_sum_fp32_cl", ea); r["vexp"] = EO.get().copy(); r["vexp_sum"] = ES.get()[:1].copy()
        D = self.t(v)
        da = self.args(self.sname("div_args"), input=D, n=1.7, dim=n)
        self.call(self.fname("pulp_div_fp32_cl"), da); r["vdiv"] = D.get().copy()
        A, Bm = i["A"], i["B"]; Hh, Ww = A.shape
        AA, BB, SS, OO = self.t(A), self.t(Bm), self.zeros(Hh), self.zeros(Hh, Ww)
        o1 = self.args(self.sname("sm_bw_op_1_args"), A=AA, B=BB, S=SS, H=Hh, W=Ww)
        self.call(nm("pulp_sm_bw_op_1"), o1); r["op1"] = SS.get().copy()
        o2 = self.args(self.sname("sm_bw_op_2_args"), A=AA, B=BB, S=SS, output=OO, H=Hh, W=Ww)
        self.call(nm("pulp_sm_bw_op_2"), o2); r["op2"] = OO.get().copy()
        if not h:
            sq = i["sq"]; d = sq.shape[0]
            SQ, SM, SO, SU = self.t(sq), self.t(sq.max(axis=1)), self.zeros(d, d), self.zeros(d)
            sha = self.args("shift_sum_args", input=SQ, sums=SU, output=SO, dim=d, dim2=d, maxes=SM)
            self.call("pulp_shift_sum_fp32_cl", sha); r["shift"] = SO.get().copy(); r["shift_sum"] = SU.get().copy()
        return r

    def transpose(self, x, axes):
        X, O = self.t(x), self.zeros(x.size)
        dims = (ctypes.c_int * x.ndim)(*x.shape); ax = (ctypes.c_int * x.ndim)(*axes)
        args = self.args(self.sname("transp_args"), in_matrix=X, out_matrix=O, dim=self.keep.hold(dims), transposed_axes=self.keep.hold(ax), n_dim=x.ndim)
        self.call("transpose" + self.sfx, args)
        return O.get().reshape([x.shape[a] for a in axes]).copy()

    def transpose_matrix(self, x):
        N, M = x.shape
        X, O = self.t(x), self.zeros(M, N)
        args = self.args(self.sname("transp_args"), in_matrix=X, out_matrix=O, N=N, M=M)
        self.call("transpose_matrix" + self.sfx, args)
        return O.get().copy()

    def broadcast_add(self, a, b):
        A, B = self.t(a), self.t(b)
        O = self.zeros(*np.broadcast_shapes(a.shape, b.shape))
        da = (ctypes.c_int * a.ndim)(*a.shape); db = (ctypes.c_int * b.ndim)(*b.shape)
        args = self.args(self.sname("array_broadcast_sum_args"), op_1=A, op_2=B, dest=O, op_1_dims=self.keep.hold(da), op_2_dims=self.keep.hold(db),
                         op_1_dims_len=a.ndim, op_2_dims_len=b.ndim)
        self.call("array_broadcast_sum_fp16" if self.half else "array_broadcast_sum_fp32", args)
        return O.get().copy()

    def pad(self, x, padL, padR, padU, padD, hwc=0):
        if hwc:
            H, W, C = x.shape; O = self.zeros(H + padU + padD, W + padL + padR, C)
        else:
            C, H, W = x.shape; O = self.zeros(C, H + padU + padD, W + padL + padR)
        X = self.t(x)
        args = self.args(self.sname("pad_args"), source=X, dest=O, C=C, H=H, W=W, T_LPAD=padL, T_RPAD=padR, T_UPAD=padU, T_DPAD=padD, HWC_lay=hwc)
        self.call("pad_tensor" + self.sfx, args)
        return O.get().copy()

    def im2row(self, x_or_dy, g, mod=0, hwc=0, fn="pulp_im2row_fp32"):
        from oracle_bind import out_hw
        Ho, Wo = out_hw(g)
        K = (g["Cout"] if mod else g["Cin"]) * g["Hk"] * g["Wk"]
        rows = g["Hin"] * g["Win"] if mod else Ho * Wo
        BUF = self.zeros(rows * K)
        Xd = self.t(x_or_dy) if not mod else self.zeros(g["Cin"], g["Hin"], g["Win"])
        dY = self.t(x_or_dy) if mod else self.zeros(g["Cout"], Ho, Wo)
        dummy = self.zeros(1)
        args = self.args(self.sname("im2col_args"), input=self.blob(Xd, dummy, C=g["Cin"], H=g["Hin"], W=g["Win"]),
                         c=self.blob(dummy, dummy, C=g["Cin"], H=g["Hk"], W=g["Wk"]), output=self.blob(dummy, dY, C=g["Cout"], H=Ho, W=Wo),
                         pBuffer=BUF, Lpad=g["padL"], Rpad=g["padR"], Upad=g["padU"], Dpad=g["padD"], mod=mod,
                         stride_w=g["sw"], stride_h=g["sh"], HWC=hwc, USE_DMA=0)
        self.call(self.fname(fn), args)
        return BUF.get().copy()

    def blocktransp(self, w, Cin, Cout, Hk, Wk, hwc=0):
        W_, BT = self.t(w), self.zeros(w.size)
        args = self.args(self.sname("blocktransp_args"), weights=W_, bt_weights=BT, Cin=Cin, Cout=Cout, Hk=Hk, Wk=Wk, HWC=hwc)
        self.call(self.fname("pulp_blocktransp_fp32"), args)
        return BT.get().reshape(w.shape).copy()
