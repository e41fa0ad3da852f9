"""The MobileBERT-style block of bench_layers.MobileBertBlock composed on the CPU from the oracle's primitives (matrix
product, layer norm forward/backward, MobileBERT attention forward/backward, GELU forward/backward, MSE): the checker for
the composition that config 4 measures.  Token-major activations [L x features]; names follow bench_layers."""
import numpy as np

F = np.float32


def run_block(o, P, X, T, heads, nffn, loss_scale, eps=1e-3):
    """o: oracle binding; P: dict of parameters (Wbi, Wbo, Wq, Wk, Wv, Wo, W1_f, W2_f, ln*_w, ln*_b); returns activations and gradients."""
    mm = lambda A, B: o.mm(np.ascontiguousarray(A, F), np.ascontiguousarray(B, F), A.shape[0], A.shape[1], B.shape[1], 0)
    ln = lambda x, n: o.layernorm_fw(np.ascontiguousarray(x, F), P[n + "_w"], P[n + "_b"], x.shape[0], x.shape[1], eps)
    L, H = X.shape; B = P["Wbi"].shape[1]
    zb = np.zeros(B, F)
    a = {}
    a["t0"] = mm(X, P["Wbi"]); a["x1"] = ln(a["t0"], "ln1")
    att = o.mobilebert(a["x1"], a["x1"], P["Wq"], P["Wk"], P["Wv"], zb, zb, zb, P["Wo"], zb, None, L, B, B, B, B, heads)
    a["att"] = att["y"]; a["r1"] = (a["x1"] + a["att"]).astype(F); a["x2"] = ln(a["r1"], "ln2")
    x = a["x2"]; ffn = []
    for f in range(nffn):
        h = mm(x, P["W1_%d" % f]); g = o.act_fw(3, h.ravel()).reshape(h.shape); out = mm(g, P["W2_%d" % f])
        r = (x + out).astype(F); xn = ln(r, "lnf_%d" % f)
        ffn.append(dict(x=x, h=h, g=g, r=r)); x = xn
    a["xf"] = x
    a["t1"] = mm(x, P["Wbo"]); a["r2"] = (X + a["t1"]).astype(F); a["Y"] = ln(a["r2"], "ln_out")
    loss, dY = o.mse(a["Y"].ravel().copy(), T.ravel().copy())
    a["loss"] = np.array([loss], F)
    # ---------------- backward (every gradient carries the loss scale, as in the block)
    G = {}
    dY = (dY * F(loss_scale)).astype(F).reshape(a["Y"].shape)
    lnb = lambda x, n, dy: o.layernorm_bw(np.ascontiguousarray(x, F), P[n + "_w"], np.ascontiguousarray(dy, F), x.shape[0], x.shape[1], eps)
    dr2, G["ln_out_w"], G["ln_out_b"] = lnb(a["r2"], "ln_out", dY)
    G["Wbo"] = mm(a["xf"].T, dr2); dx = mm(dr2, P["Wbo"].T)
    for f in reversed(range(nffn)):
        c = ffn[f]
        dr, G["lnf_%d_w" % f], G["lnf_%d_b" % f] = lnb(c["r"], "lnf_%d" % f, dx)
        G["W2_%d" % f] = mm(c["g"].T, dr); dg = mm(dr, P["W2_%d" % f].T)
        dh = o.act_bw(3, c["h"].ravel(), c["g"].ravel(), dg.ravel()).reshape(dg.shape)
        G["W1_%d" % f] = mm(c["x"].T, dh); dx = (mm(dh, P["W1_%d" % f].T) + dr).astype(F)
    dr1, G["ln2_w"], G["ln2_b"] = lnb(a["r1"], "ln2", dx)
    bw = o.mobilebert(a["x1"], a["x1"], P["Wq"], P["Wk"], P["Wv"], zb, zb, zb, P["Wo"], zb, np.ascontiguousarray(dr1, F), L, B, B, B, B, heads)
    G["Wq"], G["Wk"], G["Wv"], G["Wo"] = bw["dwq"], bw["dwk"], bw["dwv"], bw["dwo"]
    dx1 = (bw["dx"] + bw["dxb"] + dr1).astype(F)
    dt0, G["ln1_w"], G["ln1_b"] = lnb(a["t0"], "ln1", dx1)
    G["Wbi"] = mm(X.T, dt0)
    G["X"] = (mm(dt0, P["Wbi"].T) + dr2).astype(F)
    return a, G
