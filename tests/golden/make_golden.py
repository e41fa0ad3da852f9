"""Regenerates tests/golden/*.npz.  Needs the reference checkout (see --ref):

    python tests/golden/make_golden.py [--ref <reference checkout>]

* every case of tests/golden_cases.py is run through the reference's own C sources
  (oracle/_ref/libpulp_ref.so, built by `make -C oracle ref`) and stored as inputs + outputs;
* mhsa_torch_gm.npz holds the outputs of the reference's PyTorch golden model of MHSA
  (tests/test_mhsa_fp32/utils/mhsa.py, imported from the checkout) on seeded inputs.
The stored vectors are what the CPU and GPU suites compare against when the checkout is absent.
"""
import argparse
import ctypes
import os
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
TESTS = os.path.dirname(HERE)
ROOT = os.path.dirname(TESTS)
sys.path.insert(0, TESTS)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("TRAINLIB_REF", os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "..", "reference")))
    a = ap.parse_args()
    from conftest import load_pkg
    from abi_runner import AbiRunner
    import golden_cases

    subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle"), "ref", "REF=" + a.ref], stdout=subprocess.DEVNULL)
    pkg = load_pkg()
    ref = pkg.bind(ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libpulp_ref.so")))
    for name, make_inputs, run_abi, _, _ in golden_cases.CASES:
        rng = np.random.default_rng(golden_cases.case_seed(name))
        inp = make_inputs(rng)
        r = AbiRunner(pkg, ref, is_ref=True)
        out = run_abi(r, inp)
        r.close()
        blob = {"in_" + k: v for k, v in inp.items()}
        blob.update({"out_" + k: np.asarray(v) for k, v in out.items()})
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **blob)
        print("wrote", name, sorted(out))

    # PyTorch golden model of the reference's MHSA test
    import torch
    sys.path.insert(0, os.path.join(a.ref, "tests", "test_mhsa_fp32", "utils"))
    from mhsa import MultiHeadedSelfAttention
    torch.manual_seed(0)
    L, E, Fd, NH = 16, 8, 16, 2
    m = MultiHeadedSelfAttention(E, NH, Fd)
    with torch.no_grad():
        for p in (m.proj_q, m.proj_k, m.proj_v):
            p.weight.normal_(0, E ** -0.5); p.bias.normal_(0, 0.1)
        m.proj_out.weight.normal_(0, E ** -0.5)
    x = torch.randn(L, E, requires_grad=True); dy = torch.randn(L, E)
    y = m(x, L); y.backward(dy)
    f = lambda t: np.ascontiguousarray(t.detach().numpy().astype(np.float32))
    np.savez_compressed(os.path.join(HERE, "mhsa_torch_gm.npz"),
                        L=L, E=E, F=Fd, heads=NH,
                        in_x=f(x.t()), in_dy=f(dy.t()),
                        in_wq=f(m.proj_q.weight.t()), in_wk=f(m.proj_k.weight.t()), in_wv=f(m.proj_v.weight.t()), in_wo=f(m.proj_out.weight),
                        in_bq=f(m.proj_q.bias), in_bk=f(m.proj_k.bias), in_bv=f(m.proj_v.bias),
                        out_y=f(y.t()), out_dx=f(x.grad.t()), out_dwq=f(m.proj_q.weight.grad), out_dwk=f(m.proj_k.weight.grad),
                        out_dwv=f(m.proj_v.weight.grad), out_dwo=f(m.proj_out.weight.grad))
    print("wrote mhsa_torch_gm")


if __name__ == "__main__":
    main()
