"""ctypes binding of oracle/liboracle.so (the CPU restatement; checker only)."""
import ctypes
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PATH = os.path.join(ROOT, "oracle", "liboracle.so")

_f = ctypes.c_float
_i = ctypes.c_int
_l = ctypes.c_long
_p = ctypes.c_void_p


def _ptr(a):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data


class Oracle(object):
    def __init__(self, lib):
        self.lib = lib
        lib.orc_fastexp_gist.argtypes = [_f]; lib.orc_fastexp_gist.restype = _f
        lib.orc_q_rsqrt.argtypes = [_f]; lib.orc_q_rsqrt.restype = _f
        lib.orc_mse_fw.restype = _f; lib.orc_mse_fw.argtypes = [_p, _p, _i]
        lib.orc_ce_fw.restype = _f; lib.orc_ce_fw.argtypes = [_p, _p, _i]

    # scalars
    def fastexp_gist(self, x): return self.lib.orc_fastexp_gist(_f(x))
    def q_rsqrt(self, x): return self.lib.orc_q_rsqrt(_f(x))

    def mm(self, A, B, N, K, M, trans_B=0, C=None):
        acc = C is not None
        C = np.array(C, dtype=np.float32) if acc else np.zeros((N, M), np.float32)
        self.lib.orc_mm(_p(_ptr(A)), _p(_ptr(B)), _p(_ptr(C)), _i(N), _i(K), _i(M), _i(trans_B), _i(1 if acc else 0))
        return C

    def im2row(self, src, C, H, W, Hk, Wk, Ho, Wo, sh, sw, padU, padL, mode_ig=0, hwc=0, transposed=0):
        rows = H * W if mode_ig else Ho * Wo
        buf = np.zeros(rows * C * Hk * Wk, np.float32)
        self.lib.orc_im2row(_p(_ptr(src)), _p(_ptr(buf)), _i(C), _i(H), _i(W), _i(Hk), _i(Wk), _i(Ho), _i(Wo),
                            _i(sh), _i(sw), _i(padU), _i(padL), _i(mode_ig), _i(hwc), _i(transposed))
        return buf

    def blocktransp(self, w, Cin, Cout, Hk, Wk, hwc=0):
        bt = np.zeros_like(w)
        self.lib.orc_blocktransp(_p(_ptr(w)), _p(_ptr(bt)), _i(Cin), _i(Cout), _i(Hk), _i(Wk), _i(hwc))
        return bt

    @staticmethod
    def _geom(g):
        return [_i(g[k]) for k in ("Cin", "Hin", "Win", "Cout", "Hk", "Wk", "sh", "sw", "padU", "padD", "padL", "padR")]

    def conv2d_fw(self, x, w, bias, g):
        Ho, Wo = out_hw(g)
        y = np.zeros((g["Cout"], Ho, Wo), np.float32)
        self.lib.orc_conv2d_fw(_p(_ptr(x)), _p(_ptr(w)), _p(_ptr(bias)), _p(_ptr(y)), *self._geom(g))
        return y

    def conv2d_wg(self, x, dy, g, with_bias=False):
        dw = np.zeros((g["Cout"], g["Cin"], g["Hk"], g["Wk"]), np.float32)
        db = np.zeros(g["Cout"], np.float32) if with_bias else None
        self.lib.orc_conv2d_wg(_p(_ptr(x)), _p(_ptr(dy)), _p(_ptr(dw)), _p(_ptr(db)), *self._geom(g))
        return dw, db

    def conv2d_ig(self, dy, w, g):
        dx = np.zeros((g["Cin"], g["Hin"], g["Win"]), np.float32)
        self.lib.orc_conv2d_ig(_p(_ptr(dy)), _p(_ptr(w)), _p(_ptr(dx)), *self._geom(g))
        return dx

    @staticmethod
    def _dwgeom(g):
        return [_i(g[k]) for k in ("Cin", "Hin", "Win", "Hk", "Wk", "sh", "sw", "padU", "padD", "padL", "padR")]

    def dw_fw(self, x, w, g):
        Ho, Wo = out_hw(g)
        y = np.zeros((g["Cin"], Ho, Wo), np.float32)
        self.lib.orc_dw_fw(_p(_ptr(x)), _p(_ptr(w)), _p(_ptr(y)), *self._dwgeom(g))
        return y

    def dw_wg(self, x, dy, g):
        dw = np.zeros((g["Cin"], g["Hk"], g["Wk"]), np.float32)
        self.lib.orc_dw_wg(_p(_ptr(x)), _p(_ptr(dy)), _p(_ptr(dw)), *self._dwgeom(g))
        return dw

    def dw_ig(self, dy, w, g):
        dx = np.zeros((g["Cin"], g["Hin"], g["Win"]), np.float32)
        self.lib.orc_dw_ig(_p(_ptr(dy)), _p(_ptr(w)), _p(_ptr(dx)), *self._dwgeom(g))
        return dx

    def linear(self, W, x, dy, bias=None):
        out, inn = W.shape
        y = np.zeros(out, np.float32); dW = np.zeros_like(W); dx = np.zeros(inn, np.float32)
        db = np.zeros(out, np.float32) if bias is not None else None
        self.lib.orc_linear_fw(_p(_ptr(W)), _p(_ptr(x)), _p(_ptr(bias)), _p(_ptr(y)), _i(out), _i(inn))
        self.lib.orc_linear_wg(_p(_ptr(dy)), _p(_ptr(x)), _p(_ptr(dW)), _p(_ptr(db)), _i(out), _i(inn))
        self.lib.orc_linear_ig(_p(_ptr(dy)), _p(_ptr(W)), _p(_ptr(dx)), _i(out), _i(inn))
        return dict(y=y, dW=dW, dx=dx, db=db)

    def softmax_fw(self, x):
        out = np.zeros_like(x)
        self.lib.orc_softmax_fw(_p(_ptr(x)), _p(_ptr(out)), _i(x.shape[0]), _i(x.shape[1]))
        return out

    def softmax_bw(self, out, dout):
        din = np.zeros_like(out)
        self.lib.orc_softmax_bw(_p(_ptr(out)), _p(_ptr(dout)), _p(_ptr(din)), _i(out.shape[0]), _i(out.shape[1]))
        return din

    def mhsa(self, x, wq, wk, wv, bq, bk, bv, wo, dy, L, E, F, heads):
        """x, dy: E x L; weights E x F.  Returns forward tensors and all gradients."""
        z = lambda *s: np.zeros(s, np.float32)
        r = dict(q=z(F, L), k=z(F, L), v=z(F, L), softmax=z(heads, L, L), att=z(F, L), y=z(E, L))
        self.lib.orc_mhsa_fw(_p(_ptr(x)), _p(_ptr(wq)), _p(_ptr(wk)), _p(_ptr(wv)), _p(_ptr(bq)), _p(_ptr(bk)), _p(_ptr(bv)),
                             _p(_ptr(wo)), _p(_ptr(r["q"])), _p(_ptr(r["k"])), _p(_ptr(r["v"])), _p(_ptr(r["softmax"])),
                             _p(_ptr(r["att"])), _p(_ptr(r["y"])), _i(L), _i(E), _i(F), _i(heads))
        if dy is not None:
            r.update(dq=z(F, L), dk=z(F, L), dv=z(F, L), dsoftmax=z(heads, L, L), datt=z(F, L),
                     dwq=z(F, E), dwk=z(F, E), dwv=z(F, E), dwo=z(E, F), dx=z(E, L))
            self.lib.orc_mhsa_bw(_p(_ptr(x)), _p(_ptr(wq)), _p(_ptr(wk)), _p(_ptr(wv)), _p(_ptr(wo)),
                                 _p(_ptr(r["q"])), _p(_ptr(r["k"])), _p(_ptr(r["v"])), _p(_ptr(r["softmax"])), _p(_ptr(r["att"])),
                                 _p(_ptr(dy)), _p(_ptr(r["dq"])), _p(_ptr(r["dk"])), _p(_ptr(r["dv"])), _p(_ptr(r["dsoftmax"])),
                                 _p(_ptr(r["datt"])), _p(_ptr(r["dwq"])), _p(_ptr(r["dwk"])), _p(_ptr(r["dwv"])), _p(_ptr(r["dwo"])),
                                 _p(_ptr(r["dx"])), _i(L), _i(E), _i(F), _i(heads))
        return r

    def mobilebert(self, x, xb, wq, wk, wv, bq, bk, bv, wo, bo, dy, L, E, Kb, F, No, heads):
        """x: L x E, xb: L x Kb, Wq/Wk: F x Kb, Wv: F x E, Wo: No x F, dy: L x No (None: forward only)."""
        z = lambda *s: np.zeros(s, np.float32)
        r = dict(q=z(F, L), k=z(F, L), v=z(F, L), softmax=z(heads, L, L), att=z(F, L), y=z(L, No))
        P = lambda a: _p(_ptr(a))
        dims = (_i(L), _i(E), _i(Kb), _i(F), _i(No), _i(heads))
        self.lib.orc_mhsa_mobilebert_fw(P(x), P(xb), P(wq), P(wk), P(wv), P(bq), P(bk), P(bv), P(wo), P(bo),
                                        P(r["q"]), P(r["k"]), P(r["v"]), P(r["softmax"]), P(r["att"]), P(r["y"]), *dims)
        if dy is not None:
            r.update(dq=z(F, L), dk=z(F, L), dv=z(F, L), dsoftmax=z(heads, L, L), datt=z(F, L),
                     dwq=z(F, Kb), dwk=z(F, Kb), dwv=z(F, E), dwo=z(No, F), dx=z(L, E), dxb=z(L, Kb))
            self.lib.orc_mhsa_mobilebert_bw(P(x), P(xb), P(wq), P(wk), P(wv), P(wo), P(r["q"]), P(r["k"]), P(r["v"]), P(r["softmax"]), P(r["att"]),
                                            P(dy), P(r["dq"]), P(r["dk"]), P(r["dv"]), P(r["dsoftmax"]), P(r["datt"]),
                                            P(r["dwq"]), P(r["dwk"]), P(r["dwv"]), P(r["dwo"]), P(r["dx"]), P(r["dxb"]), *dims)
        return r

    def act_fw(self, kind, x, slope=0.0):
        y = np.zeros_like(x)
        self.lib.orc_act_fw(_i(kind), _p(_ptr(x)), _p(_ptr(y)), _l(x.size), _f(slope))
        return y

    def act_bw(self, kind, x, y, dy, slope=0.0):
        dx = np.zeros_like(x)
        self.lib.orc_act_bw(_i(kind), _p(_ptr(x)), _p(_ptr(y)), _p(_ptr(dy)), _p(_ptr(dx)), _l(x.size), _f(slope))
        return dx

    def instnorm(self, x, gb, dy=None):
        C = x.shape[0]; D = x.size // C
        y = np.zeros_like(x); m = np.zeros(C, np.float32); v = np.zeros(C, np.float32); s = np.zeros(C, np.float32)
        self.lib.orc_instnorm_fw(_p(_ptr(x)), _p(_ptr(y)), _p(_ptr(gb)), _p(_ptr(m)), _p(_ptr(v)), _p(_ptr(s)), _i(C), _i(D))
        r = dict(y=y, mean=m, var=v, std=s)
        if dy is not None:
            dx = np.zeros_like(x); dgb = np.zeros_like(gb)
            self.lib.orc_instnorm_bw_input(_p(_ptr(x)), _p(_ptr(dy)), _p(_ptr(dx)), _p(_ptr(gb)), _p(_ptr(m)), _p(_ptr(v)), _p(_ptr(s)), _i(C), _i(D))
            self.lib.orc_instnorm_bw_param(_p(_ptr(x)), _p(_ptr(dy)), _p(_ptr(dgb)), _p(_ptr(m)), _p(_ptr(s)), _i(C), _i(D))
            r.update(dx=dx, dgb=dgb)
        return r

    def batchnorm_fw(self, x, w, b, B, C, HW, eps):
        y = np.zeros_like(x)
        self.lib.orc_batchnorm_fw(_p(_ptr(x)), _p(_ptr(y)), _p(_ptr(w)), _p(_ptr(b)), _i(B), _i(C), _i(HW), _f(eps))
        return y

    def layernorm_fw(self, x, w, b, rows, width, eps):
        y = np.zeros_like(x)
        self.lib.orc_layernorm_fw(_p(_ptr(x)), _p(_ptr(y)), _p(_ptr(w)), _p(_ptr(b)), _i(rows), _i(width), _f(eps))
        return y

    def mm_broadcast(self, A, B):
        import ctypes
        ad = (ctypes.c_int * A.ndim)(*A.shape); bd = (ctypes.c_int * B.ndim)(*B.shape)
        out_shape = np.broadcast_shapes(A.shape[:-2], B.shape[:-2]) + (A.shape[-2], B.shape[-1])
        C = np.zeros(out_shape, np.float32)
        self.lib.orc_mm_broadcast(_p(_ptr(A)), _p(_ptr(B)), _p(_ptr(C)), ad, _i(A.ndim), bd, _i(B.ndim))
        return C

    def layernorm_bw(self, x, w, dy, rows, width, eps):
        dx = np.zeros_like(x); dw = np.zeros(width, np.float32); db = np.zeros(width, np.float32)
        self.lib.orc_layernorm_bw(_p(_ptr(x)), _p(_ptr(w)), _p(_ptr(dy)), _p(_ptr(dx)), _p(_ptr(dw)), _p(_ptr(db)), _i(rows), _i(width), _f(eps))
        return dx, dw, db

    def mse(self, y, t):
        dy = np.zeros_like(y)
        loss = self.lib.orc_mse_fw(_p(_ptr(y)), _p(_ptr(t)), _i(y.size))
        self.lib.orc_mse_bw(_p(_ptr(y)), _p(_ptr(t)), _p(_ptr(dy)), _i(y.size))
        return np.float32(loss), dy

    def ce(self, z, t):
        dz = np.zeros_like(z)
        loss = self.lib.orc_ce_fw(_p(_ptr(z)), _p(_ptr(t)), _i(z.size))
        self.lib.orc_ce_bw(_p(_ptr(z)), _p(_ptr(t)), _p(_ptr(dz)), _i(z.size))
        return np.float32(loss), dz

    def sgd(self, w, g, lr, lam=0.0):
        w = w.copy(); g = g.copy()
        self.lib.orc_sgd(_p(_ptr(w)), _p(_ptr(g)), _l(w.size), _f(lr), _f(lam))
        return w, g

    def avgpool(self, x, dy, Hk, Wk, sh, sw):
        C, H, W = x.shape
        Ho, Wo = (H - Hk + sh) // sh, (W - Wk + sw) // sw
        y = np.zeros((C, Ho, Wo), np.float32); dx = np.zeros_like(x)
        self.lib.orc_avgpool_fw(_p(_ptr(x)), _p(_ptr(y)), _i(C), _i(H), _i(W), _i(Hk), _i(Wk), _i(sh), _i(sw))
        if dy is not None:
            self.lib.orc_avgpool_bw(_p(_ptr(dy)), _p(_ptr(dx)), _i(C), _i(H), _i(W), _i(Hk), _i(Wk), _i(sh), _i(sw))
        return y, dx

    def transpose(self, x, axes):
        dims = (ctypes.c_int * x.ndim)(*x.shape); ax = (ctypes.c_int * x.ndim)(*axes)
        out = np.zeros(x.size, x.dtype)
        self.lib.orc_transpose(_p(_ptr(x)), _p(_ptr(out)), dims, ax, _i(x.ndim))
        return out.reshape([x.shape[a] for a in axes])

    def broadcast_add(self, a, b):
        da = (ctypes.c_int * a.ndim)(*a.shape); db = (ctypes.c_int * b.ndim)(*b.shape)
        out = np.zeros(np.broadcast_shapes(a.shape, b.shape), np.float32)
        self.lib.orc_broadcast_add(_p(_ptr(a)), _p(_ptr(b)), _p(_ptr(out)), da, _i(a.ndim), db, _i(b.ndim))
        return out

    def pad(self, x, padL, padR, padU, padD, hwc=0):
        if hwc:
            H, W, C = x.shape; out = np.zeros((H + padU + padD, W + padL + padR, C), np.float32)
        else:
            C, H, W = x.shape; out = np.zeros((C, H + padU + padD, W + padL + padR), np.float32)
        self.lib.orc_pad(_p(_ptr(x)), _p(_ptr(out)), _i(C), _i(H), _i(W), _i(padL), _i(padR), _i(padU), _i(padD), _i(hwc))
        return out


def out_hw(g):
    return ((g["Hin"] - g["Hk"] + g["padU"] + g["padD"]) // g["sh"] + 1,
            (g["Win"] - g["Wk"] + g["padL"] + g["padR"]) // g["sw"] + 1)


def geom(Cin, Hin, Win, Cout, k, stride=1, pad=0):
    return dict(Cin=Cin, Hin=Hin, Win=Win, Cout=Cout, Hk=k, Wk=k, sh=stride, sw=stride, padU=pad, padD=pad, padL=pad, padR=pad)


_oracle = None


def load():
    global _oracle
    if _oracle is None:
        src = os.path.join(ROOT, "oracle", "trainlib_oracle.c")
        if not os.path.exists(PATH) or os.path.getmtime(PATH) < os.path.getmtime(src):
            subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle"), "oracle"], stdout=subprocess.DEVNULL)
        _oracle = Oracle(ctypes.CDLL(PATH))
    return _oracle
