"""Stream sharding + gradient all-reduce of the batched workload, two gloo ranks on the CPU.

The ranks run the network of bench_nets.py against the reference library built from the reference sources
(the checker; the GPU library needs a GPU), each on its shard of the streams; the summed gradients and the
updated parameters must equal those of one process that owns every stream."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench_nets  # noqa: E402

TOTAL = 5   # odd on purpose: the shards differ in size


def test_shards_cover_every_stream_once():
    for total in (1, 5, 8, 4096, 4099):
        for world in (1, 2, 3, 4, 8):
            seen = []
            for r in range(world):
                first, n = bench_nets.shard_streams(total, r, world)
                seen += list(range(first, first + n))
            assert seen == list(range(total))


def _rank_main(rank, world, port, out):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        net = bench_nets.bind_net(bench_nets.NET_REF_SEQ)
        first, n = bench_nets.shard_streams(TOTAL, rank, world)

        def allreduce(g):
            t = torch.from_numpy(g)     # shares memory: the reduced sum lands in the gradient buffer
            dist.all_reduce(t)

        r = bench_nets.reference_step(net, n, first_stream=first, steps=2, allreduce=allreduce)
        np.savez(out % rank, grads=r["grads"], params=r["params"], loss=r["loss"], first=first, n=n)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(not os.path.exists(bench_nets.NET_REF_SEQ), reason="reference network library not built")
def test_two_ranks_match_one_process(tmp_path):
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]
    out = str(tmp_path / "rank%d.npz")
    mp.spawn(_rank_main, args=(2, port, out), nprocs=2, join=True)
    whole = bench_nets.reference_step(bench_nets.bind_net(bench_nets.NET_REF_SEQ), TOTAL, steps=2)
    r0, r1 = np.load(out % 0), np.load(out % 1)
    assert int(r0["n"]) + int(r1["n"]) == TOTAL and int(r1["first"]) == int(r0["n"])
    # both ranks hold the same summed gradients and the same updated parameters
    np.testing.assert_array_equal(r0["grads"], r1["grads"])
    np.testing.assert_array_equal(r0["params"], r1["params"])
    # and they are those of the single process (the sum over streams is associated differently: fp32 tolerance)
    scale = np.abs(whole["grads"]).max()
    assert np.abs(r0["grads"] - whole["grads"]).max() <= 1e-5 * scale
    assert np.abs(r0["params"] - whole["params"]).max() <= 1e-5 * np.abs(whole["params"]).max()
    np.testing.assert_allclose(np.concatenate([r0["loss"], r1["loss"]]), whole["loss"], rtol=1e-5)
