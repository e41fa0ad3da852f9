"""CPU: the oracle restatement reproduces the committed golden vectors (outputs of the reference's
own C code, and of its PyTorch golden model for MHSA) from the committed inputs."""
import glob
import os

import numpy as np
import pytest

import golden_cases

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
from metrics import assert_close, assert_exact

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load_case(name):
    z = np.load(os.path.join(GOLD, name + ".npz"))
    inp = {k[3:]: z[k] for k in z.files if k.startswith("in_")}
    out = {k[4:]: z[k] for k in z.files if k.startswith("out_")}
    return inp, out


def test_every_case_has_a_fixture():
    have = {os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLD, "*.npz"))}
    assert {c[0] for c in golden_cases.CASES} | {"mhsa_torch_gm"} <= have


@pytest.mark.parametrize("name", [c[0] for c in golden_cases.CASES])
def test_oracle_matches_golden(oracle, name):
    _, _, _, run_oracle, tol = next(c for c in golden_cases.CASES if c[0] == name)
    inp, want = load_case(name)
    got = run_oracle(oracle, inp)
    assert set(want) <= set(got), (sorted(want), sorted(got))
    for k, v in want.items():
        g = np.asarray(got[k]).reshape(v.shape)
        if tol is None:
            assert_exact(g.astype(v.dtype), v, "%s.%s" % (name, k))
        else:
            assert_close(g, v, 5e-6, "%s.%s" % (name, k))      # same order of operations: far inside the 1e-5 bar


def test_oracle_matches_torch_golden_model(oracle):
    """Second opinion for attention: the reference's PyTorch module (fastexp softmax, q_rsqrt scaling)."""
    z = np.load(os.path.join(GOLD, "mhsa_torch_gm.npz"))
    L, E, F, heads = int(z["L"]), int(z["E"]), int(z["F"]), int(z["heads"])
    r = oracle.mhsa(z["in_x"], z["in_wq"], z["in_wk"], z["in_wv"], z["in_bq"], z["in_bk"], z["in_bv"], z["in_wo"], z["in_dy"], L, E, F, heads)
    for k in ("y", "dx", "dwq", "dwk", "dwv", "dwo"):
        assert_close(r[k], z["out_" + k], 1e-5, "mhsa torch gm %s" % k)


def test_oracle_layernorm_and_gelu_backward_match_autograd(oracle):
    """the reference has no backward for layer norm and GELU: the oracle's derivatives of the reference's forward
    formulas are pinned against PyTorch autograd of the same formulas in float64"""
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(11)
    rows, width, eps = 12, 40, 1e-5
    x = rng.standard_normal((rows, width)).astype(np.float32); w = rng.standard_normal(width).astype(np.float32)
    b = rng.standard_normal(width).astype(np.float32); dy = rng.standard_normal((rows, width)).astype(np.float32)
    tx = torch.tensor(x, dtype=torch.float64, requires_grad=True); tw = torch.tensor(w, dtype=torch.float64, requires_grad=True)
    tb = torch.tensor(b, dtype=torch.float64, requires_grad=True)
    s1 = tx.sum(1, keepdim=True); s2 = (tx * tx).sum(1, keepdim=True); mean = s1 / width
    sv = torch.sqrt((s2 - 2 * s1 * mean) / width + mean * mean + eps)         # the reference's variance formula
    y = (tx - mean) / sv * tw + tb
    y.backward(torch.tensor(dy, dtype=torch.float64))
    assert np.abs(oracle.layernorm_fw(x, w, b, rows, width, eps) - y.detach().numpy()).max() <= 1e-5
    dx, dw, db = oracle.layernorm_bw(x, w, dy, rows, width, eps)
    for got, want in ((dx, tx.grad), (dw, tw.grad), (db, tb.grad)):
        want = want.numpy()
        assert np.abs(got - want).max() <= 2e-5 * max(1.0, np.abs(want).max())
    # GELU: 0.5 x (1 + clamp(pade_tanh(0.7978 (x + 0.044715 x^3))))
    xg = np.linspace(-6, 6, 4001).astype(np.float32); dyg = rng.standard_normal(xg.size).astype(np.float32)
    t = torch.tensor(xg, dtype=torch.float64, requires_grad=True)
    u = (t * t * t * 0.044715 + t) * 0.7978; u2 = u * u
    th = ((((u2 + 378.0) * u2 + 17325.0) * u2 + 135135.0) * u) / (((28.0 * u2 + 3150.0) * u2 + 62370.0) * u2 + 135135.0)
    g = 0.5 * t * (1 + torch.clamp(th, -1.0, 1.0))
    g.backward(torch.tensor(dyg, dtype=torch.float64))
    assert np.abs(oracle.act_fw(3, xg) - g.detach().numpy()).max() <= 1e-5
    got = oracle.act_bw(3, xg, oracle.act_fw(3, xg), dyg)
    assert np.abs(got - t.grad.numpy()).max() <= 1e-4 * np.abs(t.grad.numpy()).max()


def test_resnet8_golden_is_the_reference(pkg):
    """pins tests/golden/resnet8_streams_golden.npz on the reference's own C code where that is built (streams 1984-1987
    recomputed; the file's generator is tests/golden/make_resnet8_golden.py)"""
    import sys
    sys.path.insert(0, ROOT)
    import bench_nets
    if not os.path.exists(bench_nets.NET_REF_SEQ):
        pytest.skip("oracle/_ref/libresnet8_ref_seq.so not built (needs the reference checkout at build time)")
    gold = np.load(os.path.join(ROOT, "tests", "golden", "resnet8_streams_golden.npz"))
    r = bench_nets.reference_step(bench_nets.bind_net(bench_nets.NET_REF_SEQ), 4, first_stream=1984)
    assert np.array_equal(r["loss"], gold["loss_1984"][:4]) and np.array_equal(r["logits"], gold["logits_1984"][:4])
    assert gold["grads_0"].shape == gold["grads_1984"].shape == r["grads"].shape


def test_mobilebert_attention_backward_is_the_gradient_of_its_forward(oracle):
    """The reference's MobileBERT backward does not compile, so the oracle's is pinned against the chain rule written
    independently in float64 numpy (einsum over named axes) from the tensors the forward stored: P is taken as given,
    as in the training path's backward, so the Schraudolph exponential does not enter."""
    L, E, Kb, Fd, No, heads = 13, 10, 12, 16, 9, 4
    H = Fd // heads
    rng = np.random.default_rng(99)
    f = lambda *s: rng.standard_normal(s).astype(np.float32)
    x, xb, dy = f(L, E), f(L, Kb), f(L, No)
    wq, wk, wv, wo = f(Fd, Kb) / 3, f(Fd, Kb) / 3, f(Fd, E) / 3, f(No, Fd) / 4
    bq, bk, bv, bo = f(Fd) / 10, f(Fd) / 10, f(Fd) / 10, f(No) / 10
    o = oracle.mobilebert(x, xb, wq, wk, wv, bq, bk, bv, wo, bo, dy, L, E, Kb, Fd, No, heads)
    D = np.float64
    # forward pieces in float64 from the same inputs
    q = wq.astype(D) @ xb.astype(D).T + bq[:, None]; k = wk.astype(D) @ xb.astype(D).T + bk[:, None]; v = wv.astype(D) @ x.astype(D).T + bv[:, None]
    for name, want in (("q", q), ("k", k), ("v", v)):
        assert np.abs(o[name] - want).max() <= 1e-5 * np.abs(want).max(), name
    P = o["softmax"].astype(D)                                            # [head][query][key]
    vh = o["v"].astype(D).reshape(heads, H, L); qh = o["q"].astype(D).reshape(heads, H, L); kh = o["k"].astype(D).reshape(heads, H, L)
    att = np.einsum("hdk,hqk->hdq", vh, P).reshape(Fd, L)
    assert np.abs(o["att"] - att).max() <= 1e-5 * np.abs(att).max()
    y = (wo.astype(D) @ o["att"].astype(D)).T + bo[None, :]
    assert np.abs(o["y"] - y).max() <= 1e-5 * np.abs(y).max()
    # backward
    scaling = D(oracle.q_rsqrt(float(H)))
    dwo = dy.astype(D).T @ o["att"].astype(D).T                           # [n][f]
    datt = wo.astype(D).T @ dy.astype(D).T                                # [f][l]
    dah = datt.reshape(heads, H, L)
    dv = np.einsum("hdq,hqk->hdk", dah, P)
    dP = np.einsum("hdq,hdk->hqk", dah, vh)
    dS = (dP - (dP * P).sum(-1, keepdims=True)) * P * scaling
    dk = np.einsum("hdq,hqk->hdk", qh, dS); dq = np.einsum("hdk,hqk->hdq", kh, dS)
    dqf, dkf, dvf = dq.reshape(Fd, L), dk.reshape(Fd, L), dv.reshape(Fd, L)
    want = dict(dwo=dwo, datt=datt, dv=dvf, dsoftmax=dP, dk=dkf, dq=dqf, dwq=dqf @ xb.astype(D), dwk=dkf @ xb.astype(D), dwv=dvf @ x.astype(D),
                dxb=dqf.T @ wq.astype(D) + dkf.T @ wk.astype(D), dx=dvf.T @ wv.astype(D))
    for name, w in want.items():
        err = np.abs(o[name] - w).max() / np.abs(w).max()
        assert err <= 2e-5, (name, err)
