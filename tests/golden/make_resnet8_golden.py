"""Generates resnet8_streams_golden.npz: outputs of the REFERENCE's own C code (oracle/_ref/libresnet8_ref_seq.so =
pulp-trainlib_b200/nets/resnet8_streams.c built with -DNET_REFERENCE against the reference sources, sequential team,
strict fp flags) for the seeded batched workload of bench.py, step 0 (initial weights):

  loss_<a>, logits_<a>   per-stream CrossEntropy and logits of the 64 streams starting at a, a in {0, 1984, 4032}
  grads_<a>              weight gradients summed over those 64 streams, a in {0, 1984}

The GPU tests check a 2048-stream launch against streams 0-63 and 1984-2047, bench.py checks its 4096-stream launch
against streams 0-63 and 4032-4095.  Run from the repository root after `python -c "import __graft_entry__ as g; g.build()"`
on a machine that has the reference checkout (takes about a minute)."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import bench_nets  # noqa: E402

if __name__ == "__main__":
    net = bench_nets.bind_net(bench_nets.NET_REF_SEQ)
    out = {}
    for a in (0, 1984, 4032):
        r = bench_nets.reference_step(net, 64, first_stream=a)
        out["loss_%d" % a] = r["loss"]; out["logits_%d" % a] = r["logits"]
        if a != 4032:
            out["grads_%d" % a] = r["grads"]
        print("streams %d..%d: mean loss %.6f" % (a, a + 63, float(r["loss"].mean())))
    np.savez_compressed(os.path.join(ROOT, "tests", "golden", "resnet8_streams_golden.npz"), **out)
