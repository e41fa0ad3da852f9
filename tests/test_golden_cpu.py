"""CPU: the oracle restatement reproduces the committed golden vectors (outputs of the reference's
own C code, and of its PyTorch golden model for MHSA) from the committed inputs."""
import glob
import os

import numpy as np
import pytest

import golden_cases
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
