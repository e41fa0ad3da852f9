"""The batched workload of bench.py: the small ResNet of pulp-trainlib_b200/nets/resnet8_streams.c
trained on 4096 independent batch-1 streams (FW + WG-BW + IG-BW + SGD), streams sharded over the
ranks, weight gradients summed across ranks with one NCCL all-reduce per step."""
import ctypes
import json
import os
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
NETS = os.path.join(ROOT, "pulp-trainlib_b200", "nets")
NET_B200 = os.path.join(NETS, "libresnet8_b200.so")
NET_REF_MT = os.path.join(ROOT, "oracle", "_ref", "libresnet8_ref.so")
NET_REF_SEQ = os.path.join(ROOT, "oracle", "_ref", "libresnet8_ref_seq.so")
STREAMS = 4096
LR = 1e-2
F = np.float32


def bind_net(path):
    net = ctypes.CDLL(path)
    net.resnet8_param_count.restype = ctypes.c_size_t
    net.resnet8_workspace_floats.restype = ctypes.c_size_t; net.resnet8_workspace_floats.argtypes = [ctypes.c_int]
    net.resnet8_init_params.argtypes = [ctypes.c_void_p, ctypes.c_uint]
    net.resnet8_bind.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]; net.resnet8_bind.restype = ctypes.c_int
    net.resnet8_forward.argtypes = [ctypes.c_void_p] * 3
    net.resnet8_forward_host.argtypes = [ctypes.c_void_p] * 3
    net.resnet8_update.argtypes = [ctypes.c_float]
    net.resnet8_logits.restype = ctypes.c_void_p
    net.resnet8_flops_per_stream.restype = ctypes.c_double
    return net


def synthetic_batch(n, first_stream=0):
    """images ~ N(0,1) [n,3,32,32], labels uniform over 10 classes as one-hot rows; keyed by stream index"""
    img = np.empty((n, 3, 32, 32), F); lab = np.zeros((n, 10), F)
    for s in range(n):
        rng = np.random.default_rng(1000003 + first_stream + s)
        img[s] = rng.standard_normal((3, 32, 32)).astype(F)
        lab[s, rng.integers(0, 10)] = 1
    return img, lab


def shard_streams(total, rank, world):
    """Contiguous block of streams owned by `rank`: (first stream, count).  The first total % world ranks take one more."""
    base, extra = divmod(total, world)
    return rank * base + min(rank, extra), base + (1 if rank < extra else 0)


def host_params(net, seed=0):
    p = np.zeros(net.resnet8_param_count(), F)
    net.resnet8_init_params(p.ctypes.data, seed)
    return p


def reference_step(net_ref, n, first_stream=0, lr=LR, params=None, steps=1, allreduce=None):
    """Run the same C network against the reference library on the host; returns dict of results.
    `allreduce(array)` (in place) stands where the GPU arm sums the weight gradients over the ranks."""
    p = host_params(net_ref) if params is None else params.copy()
    g = np.zeros_like(p)
    ws = np.zeros(net_ref.resnet8_workspace_floats(n), F)
    ws[::1024] = 0                                                  # touch every page now, not inside the timed steps
    img, lab = synthetic_batch(n, first_stream)
    loss = np.zeros(n, F)
    assert net_ref.resnet8_bind(n, p.ctypes.data, g.ctypes.data, ws.ctypes.data) == 0
    t0 = time.perf_counter()
    for _ in range(steps):
        net_ref.resnet8_forward(img.ctypes.data, lab.ctypes.data, loss.ctypes.data)
        net_ref.resnet8_backward()
        if allreduce is not None:
            allreduce(g)
        grads = g.copy()
        net_ref.resnet8_update(lr)
    dt = (time.perf_counter() - t0) / steps
    logits = np.ctypeslib.as_array(ctypes.cast(net_ref.resnet8_logits(), ctypes.POINTER(ctypes.c_float)), shape=(n, 10)).copy()
    return dict(loss=loss, logits=logits, grads=grads, params=p, seconds_per_step=dt)


class ResNet8Streams(object):
    name = "c5_resnet8_4096_streams_fp32_fw_bw_sgd"

    def __init__(self, pkg, lib):
        self.pkg, self.lib = pkg, lib

    # ------------------------------------------------------------------ GPU arm
    def run(self, args, rank, world, dist):
        from bench import ClockSampler, peaks
        pkg, lib = self.pkg, self.lib
        net = bind_net(NET_B200)
        total = int(os.environ.get("TRAINLIB_BENCH_STREAMS", STREAMS))
        first, n = shard_streams(total, rank, world)
        torch = None
        if world > 1:
            import torch
            lib.trainlib_set_stream(ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        P = net.resnet8_param_count()
        hp = host_params(net)
        if torch is not None:
            t_params = torch.from_numpy(hp).cuda(); t_grads = torch.zeros(P, device="cuda")
            d_params, d_grads = t_params.data_ptr(), t_grads.data_ptr()
        else:
            b_params = pkg.DeviceBuffer(lib, hp); b_grads = pkg.DeviceBuffer(lib, nbytes=4 * P)
            d_params, d_grads = b_params.ptr, b_grads.ptr
        ws = pkg.DeviceBuffer(lib, nbytes=4 * net.resnet8_workspace_floats(n)); ws.zero()
        img, lab = synthetic_batch(n, first)
        d_img, d_lab = pkg.DeviceBuffer(lib, img), pkg.DeviceBuffer(lib, lab)
        d_loss = pkg.DeviceBuffer(lib, nbytes=4 * n)
        assert net.resnet8_bind(n, d_params, d_grads, ws.ptr) == 0
        fused = not getattr(args, "no_fusion", False)
        net.resnet8_set_fusion(1 if fused else 0)

        loss_check = self.check_first_forward(net, d_img, d_lab, d_loss, first, n, total)

        graph = [None]

        def step():
            if graph[0]:
                lib.trainlib_graph_launch(graph[0])      # forward + backward, recorded once below
            else:
                net.resnet8_forward(d_img.ptr, d_lab.ptr, d_loss.ptr)
                net.resnet8_backward()
            if torch is not None:
                dist.all_reduce(t_grads)
            net.resnet8_update(LR)

        def sync():
            lib.trainlib_synchronize()
            if torch is not None:
                torch.cuda.synchronize(); dist.barrier()

        sampler = ClockSampler(lib.trainlib_device()); sampler.start()       # sampled from the warm-up on: the GPU is under the same load
        for _ in range(args.warmup):
            step()
        sync(); pkg.check(lib)
        if not getattr(args, "no_graph", False):
            # the forward and backward pass of one step as a CUDA graph of the very same entry-point calls
            lib.trainlib_graph_begin()
            net.resnet8_forward(d_img.ptr, d_lab.ptr, d_loss.ptr); net.resnet8_backward()
            graph[0] = lib.trainlib_graph_end()
            pkg.check(lib)
            step(); sync(); pkg.check(lib)
        l0 = lib.trainlib_kernel_launches()
        sync()
        lib.trainlib_timer_start()
        for _ in range(args.steps):
            step()
        ms_total = lib.trainlib_timer_stop_ms()
        sync()
        launches = lib.trainlib_kernel_launches() - l0
        clocks = sampler.stop()
        pkg.check(lib)
        if torch is not None:
            t = torch.tensor([ms_total], device="cuda"); dist.all_reduce(t, op=dist.ReduceOp.MAX); ms_total = float(t.item())
        ms_step = ms_total / args.steps
        loss_host = d_loss.download(F, (n,))

        # end to end: the batch starts in pinned host memory every step, the losses come back
        from bench import pinned_like
        h_img, h_lab, h_loss = pinned_like(pkg, lib, img), pinned_like(pkg, lib, lab), pinned_like(pkg, lib, np.zeros(n, F))

        if graph[0]:
            # Two device copies of the batch, used in turn; per copy one CUDA graph of forward + backward.  A step uploads the
            # NEXT step's batch on the copy stream (trainlib_memcpy_h2d_overlapped) while its own kernels run, then reads its
            # losses back (blocking).  Every step still moves one batch up and one loss vector down inside the timed region.
            slots = []
            for sidx in range(2):
                di, dl = pkg.DeviceBuffer(lib, nbytes=img.nbytes), pkg.DeviceBuffer(lib, nbytes=lab.nbytes)
                lib.trainlib_memcpy_h2d(di.ptr, h_img.ctypes.data, img.nbytes); lib.trainlib_memcpy_h2d(dl.ptr, h_lab.ctypes.data, lab.nbytes)
                lib.trainlib_graph_begin()
                net.resnet8_forward(di.ptr, dl.ptr, d_loss.ptr); net.resnet8_backward()
                slots.append((di, dl, lib.trainlib_graph_end()))
                pkg.check(lib)
            state = {"i": 0}

            def upload(sidx):
                lib.trainlib_memcpy_h2d_overlapped(slots[sidx][0].ptr, h_img.ctypes.data, img.nbytes, sidx)
                lib.trainlib_memcpy_h2d_overlapped(slots[sidx][1].ptr, h_lab.ctypes.data, lab.nbytes, sidx)

            def step_e2e():
                sidx = state["i"] & 1; state["i"] += 1
                lib.trainlib_graph_launch(slots[sidx][2])
                lib.trainlib_mark_consumed(sidx)
                if torch is not None:
                    dist.all_reduce(t_grads)
                net.resnet8_update(LR)
                upload(sidx ^ 1)
                lib.trainlib_memcpy_d2h(h_loss.ctypes.data, d_loss.ptr, 4 * n)
            upload(0)
        else:
            def step_e2e():
                net.resnet8_forward_host(h_img.ctypes.data, h_lab.ctypes.data, h_loss.ctypes.data)
                net.resnet8_backward()
                if torch is not None:
                    dist.all_reduce(t_grads)
                net.resnet8_update(LR)

        for _ in range(2):
            step_e2e()
        sync()
        lib.trainlib_timer_start()
        e2e_steps = max(3, args.steps // 2)
        for _ in range(e2e_steps):
            step_e2e()
        e2e_ms = lib.trainlib_timer_stop_ms()
        sync()
        if torch is not None:
            t = torch.tensor([e2e_ms], device="cuda"); dist.all_reduce(t, op=dist.ReduceOp.MAX); e2e_ms = float(t.item())
        e2e_ms /= e2e_steps
        pkg.check(lib)

        # the same step with no pipelining at all: the entry points get HOST pointers for the batch and the losses, so the
        # library stages the upload before the first kernel and the read-back after the last one of the call, in line
        def step_strict():
            net.resnet8_forward_host(h_img.ctypes.data, h_lab.ctypes.data, h_loss.ctypes.data)
            net.resnet8_backward()
            if torch is not None:
                dist.all_reduce(t_grads)
            net.resnet8_update(LR)
        step_strict(); sync()
        lib.trainlib_timer_start()
        for _ in range(3):
            step_strict()
        strict_ms = lib.trainlib_timer_stop_ms()
        sync()
        if torch is not None:
            t = torch.tensor([strict_ms], device="cuda"); dist.all_reduce(t, op=dist.ReduceOp.MAX); strict_ms = float(t.item())
        strict_ms /= 3
        pkg.check(lib)

        # per-kernel durations of one more step, CUDA events around every launch on the library stream
        lib.trainlib_profile(1)
        net.resnet8_forward(d_img.ptr, d_lab.ptr, d_loss.ptr); net.resnet8_backward(); net.resnet8_update(LR)
        lib.trainlib_profile(0)
        table = pkg.profile_table(lib, flops=True)
        pkg.check(lib)
        if rank != 0:
            return None
        pk = peaks()
        flops_step = net.resnet8_flops_per_stream() * total
        line = {"metric": "train_step_samples_per_s", "value": total / (ms_step * 1e-3), "unit": "samples/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "tflops": flops_step / (ms_step * 1e-3) / 1e12,
                "config": {"workload": self.name, "streams_total": total, "streams_per_gpu": n, "lr": LR,
                           "l2": "per-step working set (%.1f GB) exceeds L2; no flush needed" % (4e-9 * net.resnet8_workspace_floats(n)),
                           "parallelism": "streams sharded over %d rank(s); one NCCL all-reduce of %d gradient floats per step" % (world, P),
                           "replay": "forward + backward replayed as a CUDA graph of the entry-point calls" if graph[0] else "entry-point calls",
                           "calls": "norm + residual sum + ReLU and the shortcut gradient joins as one library call each (same bits as the separate calls; --no-fusion issues the reference's separate calls)" if fused
                                    else "the reference's separate calls for norm, residual sum, ReLU and gradient joins (--no-fusion)"},
                "gpu_launches": int(launches), "clocks": clocks, "mean_loss": float(loss_host.mean()), "loss_check": loss_check,
                "e2e": {"value": total / (e2e_ms * 1e-3), "unit": "samples/s", "ms_per_step": e2e_ms,
                        "h2d_bytes_per_step": int(img.nbytes + lab.nbytes), "d2h_bytes_per_step": int(4 * n),
                        "how": "upload of the next batch overlapped with this step's kernels (two device slots), losses read back every step" if graph[0] else "host-pointer entry points",
                        "strict": {"value": total / (strict_ms * 1e-3), "unit": "samples/s", "ms_per_step": strict_ms,
                                   "how": "host pointers handed to the reference's entry points: staging copies in line with the kernels, no graph, no overlap"}},
                "roofline": self.roofline(table, n, pk),
                "kernel_table": [{"kernel": k, "launches": c, "ms": round(ms, 4), "gflop": round(fl * 1e-9, 2)} for k, c, ms, fl in table[:40]]}
        if world == 1 and not args.no_cpu_baseline and os.path.exists(NET_REF_MT):
            line["cpu_baseline"] = self.cpu_baseline()
        return line

    def check_first_forward(self, net, d_img, d_lab, d_loss, first, n, total):
        """One forward pass with the initial weights, before anything is timed: the per-stream losses of the first and the
        last 64 streams of the job must equal the reference's own C code (tests/golden/resnet8_streams_golden.npz, written
        by tests/golden/make_resnet8_golden.py) to 1e-5 of the largest loss.  Each rank checks the windows that fall into
        its shard; a mismatch stops the benchmark, so a printed throughput always belongs to a correct forward pass."""
        path = os.path.join(ROOT, "tests", "golden", "resnet8_streams_golden.npz")
        if not os.path.exists(path):
            return {"checked_streams": 0, "note": "golden file missing"}
        gold = np.load(path)
        net.resnet8_forward(d_img.ptr, d_lab.ptr, d_loss.ptr)
        self.lib.trainlib_synchronize(); self.pkg.check(self.lib)
        assert self.lib.trainlib_tc_status() == 0, "a bounded tensor-core wait gave up: id %d" % self.lib.trainlib_tc_status()
        loss = d_loss.download(F, (n,))
        checked, worst = 0, 0.0
        for a in (0, total - 64):
            key = "loss_%d" % a
            if key in gold.files and a >= first and a + 64 <= first + n:
                want = gold[key]; got = loss[a - first:a - first + 64]
                err = float(np.abs(got.astype(np.float64) - want).max() / np.abs(want).max())
                if not (err <= 1e-5):
                    raise RuntimeError("first-step loss of streams %d..%d differs from the reference: rel err %.3e" % (a, a + 63, err))
                checked += 64; worst = max(worst, err)
        return {"checked_streams": checked, "max_rel_err": worst, "bar": 1e-5, "against": "reference C code, per-stream CrossEntropy of the first and last 64 streams, initial weights"}

    # kernel families of the step: template variants (plane sizes, tile widths) and the kernels that share one job count as one
    FAMILIES = (
        ("conv_fw_ig_tensor", ("conv_mn_kernel", "conv_tc_kernel"), "tensor",
         "forward of the 7 3x3 convolutions and their input gradients as tcgen05 3xTF32 implicit GEMMs (useful FLOP: zeros of a dilated dY are not counted)"),
        ("conv_wg_tensor", ("conv_wgt_kernel",), "tensor", "weight gradient of the stride-1 3x3 convolutions with 32+ channels as a tcgen05 3xTF32 pixel-contraction GEMM"),
        ("conv_wg_ffma", ("conv_wg3x3_partial_kernel", "conv_wg_partial_kernel", "conv_wg_direct_kernel"), "ffma", "weight gradient of the other convolutions, fp32 FFMA"),
        ("conv_1x1_strided", ("conv1x1s_mma_kernel", "conv1x1s_wg_kernel", "conv1x1_strided_ig_kernel"), "hbm",
         "forward, weight gradient and in-place input gradient of the two 1x1 stride-2 shortcut convolutions: 2 FLOP per byte, bound by memory traffic and instruction issue"),
        ("conv_fw_ig_ffma", ("conv_fw_kernel", "conv_ig_kernel"), "ffma", "convolutions on the FFMA path"),
    )
    # DRAM traffic of one launch from ncu captures at 512 streams (bytes read + written inside the launch), keyed by
    # family; scaled by the stream count, which is exact here: every stream brings its own planes
    NCU_TRAFFIC_512 = {
        # conv_mn_kernel<3, 1>, 16 -> 16 forward at 1024 streams: 67.17 MB read (= the layer's input) + 19.21 MB written
        # inside the launch (the rest of the 67.1 MB output was still dirty in L2 when the kernel ended); halved to 512
        "conv_fw_ig_tensor": {"bytes": 0.5 * (67.17e6 + 19.21e6),
                              "note": "per launch of the 16->16 32x32 forward convolution (conv_mn_kernel<3,1>), ncu at 1024 streams scaled by streams; "
                                      "reads = the layer's input bytes (65 536 B per stream), no re-reads; algorithmic bytes of that launch are 65 536 B in + 65 536 B out per stream"},
    }

    def roofline(self, table, n, pk):
        """The kernel family that takes most of the profiled step, against the bound that limits it.  FLOPs are the useful
        ones the library credits to each launch (2 per multiply-add of the operator's definition), times are CUDA events
        around every launch of one step.  `frac` is against the sustained peak (the kernels run inside a long step under
        the power cap); `frac_of_burst` is the same figure against the burst peak.  `families` lists the others."""
        if not table:
            return None
        base = {}
        for name, count, ms, fl in table:
            key = name.strip("()").split("<")[0]
            c, t, f = base.get(key, (0, 0.0, 0.0))
            base[key] = (c + count, t + ms, f + fl)
        total_ms = sum(r[2] for r in table)
        fams, used = [], set()
        for fam, members, bound, what in self.FAMILIES:
            c = sum(base[m][0] for m in members if m in base); t = sum(base[m][1] for m in members if m in base); f = sum(base[m][2] for m in members if m in base)
            used.update(members)
            if c:
                fams.append({"family": fam, "kernels": [m for m in members if m in base], "bound": bound, "launches_per_step": c, "ms_per_step": t, "flops": f, "work": what})
        for key, (c, t, f) in base.items():
            if key not in used:
                fams.append({"family": key, "kernels": [key], "bound": "hbm", "launches_per_step": c, "ms_per_step": t, "flops": 0.0, "work": "bandwidth-bound"})
        # fp32 on the tensor cores is 3xTF32: one third of the TF32 rate, TF32 = half the bf16 rate
        tensor_sus, tensor_burst = pk["bf16_tflops_sustained"] / 6.0, pk["bf16_tflops"] / 6.0
        ffma_peak = 72.8
        for f in fams:
            f["share_of_kernel_time"] = f["ms_per_step"] / total_ms if total_ms else None
            if f["bound"] == "hbm":
                continue
            f["achieved"] = f["flops"] / (f["ms_per_step"] * 1e-3) / 1e12 if f["ms_per_step"] > 0 else None
            f["unit"] = "TFLOP/s"
            if f["bound"] == "tensor":
                f.update({"peak": tensor_sus, "peak_burst": tensor_burst, "frac": f["achieved"] / tensor_sus, "frac_of_burst": f["achieved"] / tensor_burst,
                          "peak_note": "3xTF32-effective fp32 peak = measured bf16 / 6: sustained figure (kernels timed inside a long step), burst beside it"})
            else:
                f.update({"peak": ffma_peak, "frac": f["achieved"] / ffma_peak, "peak_note": "FFMA peak of this part: 125 MAC/clk/SM x 148 SMs x 1965 MHz"})
        fams.sort(key=lambda f: -f["ms_per_step"])
        compute = [f for f in fams if f["bound"] != "hbm"]
        top = dict(compute[0] if compute else fams[0])
        top["kernel"] = "+".join(top.pop("kernels"))
        top["algorithmic_flops"] = top.pop("flops")
        tr = self.NCU_TRAFFIC_512.get(top["family"])
        top["traffic"] = tr["bytes"] * n / 512.0 if tr else None
        if tr:
            top["traffic_note"] = tr["note"]
        top["peak_source"] = pk["source"]
        top["families"] = [{k: (round(v, 4) if isinstance(v, float) else v) for k, v in f.items() if k not in ("work", "peak_note", "unit")} for f in fams[:10] if f["family"] != top["family"]]
        return top

    # ------------------------------------------------------------------ reference arm (host cores)
    @staticmethod
    def _ref_worker(job):
        first, n, steps = job
        net = bind_net(NET_REF_MT)
        reference_step(net, min(n, 32), first_stream=first, steps=1)   # warm-up (code pages, thread team start)
        t0 = time.perf_counter()
        reference_step(net, n, first_stream=first, steps=steps)
        return time.perf_counter() - t0

    def _reference_throughput(self, per_proc=128, steps=1, total=None):
        """The reference library parallelises one call over a team of 8 threads (NUM_CORES is a compile-time constant of its
        sources).  Streams are independent, so all host cores are used by running cpu_count // 8 processes side by side, each
        with its own team on its own slice of the sample; throughput = streams finished / wall time of the slowest."""
        import multiprocessing as mp
        procs = max(1, (os.cpu_count() or 8) // 8)
        if total is not None:                       # the whole job, split into one contiguous block of streams per process
            jobs = [shard_streams(total, i, procs) + (steps,) for i in range(procs)]
        else:
            jobs = [(i * per_proc, per_proc, steps) for i in range(procs)]
        if procs == 1:
            times = [self._ref_worker(jobs[0])]
        else:
            with mp.get_context("fork").Pool(procs) as pool:
                times = pool.map(ResNet8Streams._ref_worker, jobs)
        wall = max(times)
        done = sum(j[1] for j in jobs)
        return {"samples_per_s": done * steps / wall, "procs": procs, "cores": 8 * procs, "sample": done, "steps": steps, "wall_s": wall}

    def cpu_baseline(self, sample=512, steps=1):
        r = self._reference_throughput(sample, steps)
        return {"value": r["samples_per_s"], "unit": "samples/s", "cores": r["cores"], "kind": "reference",
                "sample": "%d of the %d streams (%d processes x %d streams, pthread team of 8 each), %d step(s), reference C sources" % (r["sample"], STREAMS, r["procs"], sample, steps),
                "wall_s": r["wall_s"]}

    def run_reference(self, ref_lib, args):
        if not os.path.exists(NET_REF_MT):
            return {"unavailable": "oracle/_ref/libresnet8_ref.so was not built (needs the reference checkout at build time)", "value": None, "unit": "samples/s"}
        # every timed step is the whole job: all 4096 streams once through the reference's code (about 20 s on 16 cores)
        steps = max(1, min(args.steps, 2))
        r = self._reference_throughput(steps=steps, total=STREAMS)
        v = r["samples_per_s"]
        return {"metric": "train_step_samples_per_s", "value": v, "unit": "samples/s", "ms_per_step": 1e3 * STREAMS / v, "dtype": "f32",
                "config": {"workload": self.name, "streams_total": STREAMS, "streams_per_step": r["sample"], "same_config": r["sample"] == STREAMS, "timed_steps": steps},
                "cpu_baseline": {"value": v, "unit": "samples/s", "cores": r["cores"], "kind": "reference",
                                 "sample": "all %d streams per step (%d timed step(s), %.1f s each): %d processes side by side, each with the reference's pthread "
                                           "team of 8 on its own block of streams" % (r["sample"], steps, r["wall_s"] / steps, r["procs"])}}
