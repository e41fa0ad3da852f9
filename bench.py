#!/usr/bin/env python
"""Benchmark of the matmul-centred training step (FW + WG-BW + IG-BW) through the C ABI.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config c5|c2|c1|c3] [--impl ours|reference]

One JSON line on stdout (rank 0).  `value` is measured with all tensors resident in HBM;
`e2e` is the same step through the reference-facing C ABI with HOST buffers (pinned), so the
host<->device copies are inside the timed region.  `--impl reference` times the reference's own
C code (oracle/_ref/libpulp_ref_mt.so, pthread team of 8) on the host cores on a bounded sample.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
from __graft_entry__ import load_pkg  # noqa: E402

F = np.float32
REF_MT = os.path.join(ROOT, "oracle", "_ref", "libpulp_ref_mt.so")
REF_MT_CORES = 8


def peaks():
    p = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            j = json.load(open(path))
            p.update({k: j[k] for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained") if k in j})
            p["source"] = "measured"
        except Exception:
            pass
    return p


class ClockSampler(object):
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits", "-lms", "25"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for l in self.lines:
            f = [x.strip() for x in l.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------ workloads
class LinearSweep(object):
    """config 2: Linear FW + WG + IG at batch 1 over (in,out) in {(256,256),(1024,1024),(4096,1024),(1024,4096)}."""
    SHAPES = [(256, 256), (1024, 1024), (4096, 1024), (1024, 4096)]
    name = "c2_linear_sweep_fw_wg_ig_batch1"
    use_graph = True

    def __init__(self, pkg, lib, half):
        self.pkg, self.lib, self.half = pkg, lib, half
        self.dt = np.float16 if half else np.float32
        self.es = 2 if half else 4
        self.flops = sum(5.0 * i * o for i, o in self.SHAPES)
        self.bytes = sum(3.0 * i * o * self.es for i, o in self.SHAPES)
        self.units = 1
        self.keep = pkg.Keep()
        self.sfx = "_fp16" if half else ""

    def _inputs(self, rng, inn, out):
        return ((rng.standard_normal((out, inn)) / np.sqrt(inn)).astype(self.dt), rng.standard_normal(inn).astype(self.dt), rng.standard_normal(out).astype(self.dt))

    def _args(self, W, x, dy, y, dW, dx, inn, out):
        pk, k = self.pkg, self.keep
        b = lambda d, g, dim: pk.make_blob(k, d, g, dim=dim, W=dim, half=self.half)
        one = np.zeros(1, self.dt) if not isinstance(W, int) else W
        return pk.make_args(k, "Linear_args" + self.sfx, input=b(x, dx, inn), coeff=pk.make_blob(k, W, dW, C=1, H=out, W=inn, half=self.half),
                            bias=b(one, one, out), output=b(y, dy, out), skip_wg_grad=0, skip_in_grad=0, use_biases=0)

    def setup_device(self):
        rng = np.random.default_rng(2)
        self.dev, self.args_dev = [], []
        for inn, out in self.SHAPES:
            W, x, dy = self._inputs(rng, inn, out)
            bufs = [self.pkg.DeviceBuffer(self.lib, a) for a in (W, x, dy)] + [self.pkg.DeviceBuffer(self.lib, nbytes=n * self.es) for n in (out, out * inn, inn)]
            self.dev.append(bufs)
            self.args_dev.append(self._args(*[b.ptr for b in bufs], inn, out))
        self.flush = self.pkg.DeviceBuffer(self.lib, nbytes=256 << 20)

    def l2_flush(self):
        self.lib.trainlib_memset(self.flush.ptr, 1, self.flush.nbytes)

    def step_device(self):
        for a in self.args_dev:
            p = ctypes.byref(a)
            getattr(self.lib, "pulp_linear_%s_fw_cl" % ("fp16" if self.half else "fp32"))(p)
            getattr(self.lib, "pulp_linear_%s_bw_cl" % ("fp16" if self.half else "fp32"))(p)      # weight and input gradient

    def setup_host(self, lib):
        """host-pointer arguments (pinned when our library provides the allocator)"""
        rng = np.random.default_rng(2)
        self.host, self.args_host = [], []
        for inn, out in self.SHAPES:
            W, x, dy = self._inputs(rng, inn, out)
            arrs = [W, x, dy, np.zeros(out, self.dt), np.zeros((out, inn), self.dt), np.zeros(inn, self.dt)]
            if hasattr(lib, "trainlib_malloc_host"):
                arrs = [pinned_like(self.pkg, lib, a) for a in arrs]
            self.host.append(arrs)
            self.args_host.append(self._args(*arrs, inn, out))
        self.h2d = sum((2.0 * i * o + 2 * i + 2 * o) * self.es for i, o in self.SHAPES)
        self.d2h = sum((o + i * o + i) * self.es for i, o in self.SHAPES)

    def step_host(self, lib):
        for a in self.args_host:
            p = ctypes.byref(a)
            getattr(lib, "pulp_linear_%s_fw_cl" % ("fp16" if self.half else "fp32"))(p)
            getattr(lib, "pulp_linear_%s_bw_cl" % ("fp16" if self.half else "fp32"))(p)           # weight and input gradient

    def metric(self, ms):
        return {"metric": "train_step_tflops", "unit": "TFLOP/s", "value": self.flops / (ms * 1e-3) / 1e12}

    def roofline(self, ms, pk):
        gbs = self.bytes / (ms * 1e-3) / 1e9
        return {"bound": "hbm", "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": gbs / pk["hbm_gbs"], "traffic": None,
                "peak_source": pk["source"], "kernel": "linear_fw_kernel + linear_bw_fused_kernel (whole step)", "algorithmic_bytes": self.bytes}


class MmSweep(object):
    """`mm` / `mm_fp16` (C = A B, matMul_args) on square shapes: the tensor-core GEMM of the matmul family against
    the tensor roofline.  Not one of the numbered configs; `--config mm`."""
    SHAPES = [1024, 2048, 4096]
    name = "mm_square_1024_2048_4096"

    def __init__(self, pkg, lib, half):
        self.pkg, self.lib, self.half = pkg, lib, half
        self.dt = np.float16 if half else np.float32
        self.es = 2 if half else 4
        self.flops = sum(2.0 * n ** 3 for n in self.SHAPES)
        self.keep = pkg.Keep()
        self.fn = "mm_fp16" if half else "mm"

    def _args(self, A, B, C, n):
        return self.pkg.make_args(self.keep, "matMul_args" + ("_fp16" if self.half else ""), A=A, B=B, C=C, N=n, K=n, M=n, trans_B=0, USE_BIASES=0)

    def _inputs(self, rng, n):
        return (rng.standard_normal((n, n)) / np.sqrt(n)).astype(self.dt), rng.standard_normal((n, n)).astype(self.dt)

    def setup_device(self):
        rng = np.random.default_rng(3)
        self.dev, self.args_dev = [], []
        for n in self.SHAPES:
            A, B = self._inputs(rng, n)
            bufs = [self.pkg.DeviceBuffer(self.lib, A), self.pkg.DeviceBuffer(self.lib, B), self.pkg.DeviceBuffer(self.lib, nbytes=n * n * self.es)]
            self.dev.append(bufs)
            self.args_dev.append(self._args(*[b.ptr for b in bufs], n))
        self.flush = self.pkg.DeviceBuffer(self.lib, nbytes=256 << 20)

    def l2_flush(self):
        self.lib.trainlib_memset(self.flush.ptr, 1, self.flush.nbytes)

    def step_device(self):
        for a in self.args_dev:
            getattr(self.lib, self.fn)(ctypes.byref(a))

    def setup_host(self, lib):
        rng = np.random.default_rng(3)
        self.host, self.args_host = [], []
        for n in self.SHAPES:
            A, B = self._inputs(rng, n)
            arrs = [A, B, np.zeros((n, n), self.dt)]
            if hasattr(lib, "trainlib_malloc_host"):
                arrs = [pinned_like(self.pkg, lib, a) for a in arrs]
            self.host.append(arrs)
            self.args_host.append(self._args(*arrs, n))
        self.h2d = sum(3.0 * n * n * self.es for n in self.SHAPES)
        self.d2h = sum(1.0 * n * n * self.es for n in self.SHAPES)

    def step_host(self, lib):
        for a in self.args_host:
            getattr(lib, self.fn)(ctypes.byref(a))

    def metric(self, ms):
        return {"metric": "mm_tflops", "unit": "TFLOP/s", "value": self.flops / (ms * 1e-3) / 1e12}

    def per_shape(self, reps=5):
        """device time of each shape alone (inputs resident, `reps` launches back to back after one warm-up)"""
        out = []
        for n, a in zip(self.SHAPES, self.args_dev):
            getattr(self.lib, self.fn)(ctypes.byref(a))
            self.lib.trainlib_synchronize()
            self.lib.trainlib_timer_start()
            for _ in range(reps):
                getattr(self.lib, self.fn)(ctypes.byref(a))
            ms = self.lib.trainlib_timer_stop_ms() / reps
            out.append({"n": n, "ms": ms, "tflops": 2.0 * n ** 3 / (ms * 1e-3) / 1e12})
        return out

    def roofline(self, ms, pk):
        shapes = self.per_shape()
        big = shapes[-1]
        peak = pk["bf16_tflops_sustained"] if self.half else pk["bf16_tflops_sustained"] / 6.0
        return {"bound": "tensor", "achieved": big["tflops"], "peak": peak, "unit": "TFLOP/s", "frac": big["tflops"] / peak, "traffic": None,
                "peak_source": pk["source"], "kernel": "gemm_tma_kernel + pack_kmajor_kernel, %d^3" % big["n"], "algorithmic_flops": 2.0 * big["n"] ** 3,
                "per_shape": shapes, "sweep_tflops": self.flops / (ms * 1e-3) / 1e12,
                "peak_note": "measured sustained bf16 (fp16 operands)" if self.half else "3xTF32-effective fp32 peak = measured sustained bf16 / 6"}


_pinned = []


def pinned_like(pkg, lib, a):
    """numpy array over pinned host memory from the library's allocator"""
    ptr = lib.trainlib_malloc_host(max(a.nbytes, 16))
    pkg.check(lib)
    buf = (ctypes.c_char * a.nbytes).from_address(ptr)
    out = np.frombuffer(buf, dtype=a.dtype).reshape(a.shape)
    out[...] = a
    _pinned.append((ptr, buf))
    return out


def make_workload(cfg, pkg, lib, dtype):
    if cfg == "c2":
        return LinearSweep(pkg, lib, dtype == "fp16")
    if cfg == "c1":
        from bench_layers import ConvStep
        return ConvStep(pkg, lib)
    if cfg == "c3":
        from bench_layers import MhsaStep
        return MhsaStep(pkg, lib)
    if cfg == "c4":
        from bench_layers import MobileBertBlock
        return MobileBertBlock(pkg, lib, dtype != "fp32")
    if cfg == "mm":
        return MmSweep(pkg, lib, dtype == "fp16")
    if cfg == "c5":
        from bench_nets import ResNet8Streams
        return ResNet8Streams(pkg, lib)
    raise SystemExit("unknown --config %s" % cfg)


# ------------------------------------------------------------------------------------------------ runs
def time_host_lib(wl, lib, steps, warmup):
    wl.setup_host(lib)
    for _ in range(warmup):
        wl.step_host(lib)
    ts = []
    for _ in range(steps):
        t0 = time.perf_counter(); wl.step_host(lib); ts.append(time.perf_counter() - t0)
    return 1e3 * float(np.mean(ts))


def run_reference(args, pkg):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    if not os.path.exists(REF_MT):
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libpulp_ref_mt.so was not built (needs the reference checkout at build time)"}))
        return
    ref = pkg.bind(ctypes.CDLL(REF_MT))
    wl = make_workload(args.config, pkg, ref, args.dtype)
    if getattr(wl, "no_reference", None):
        print(json.dumps({"impl": "reference", "unavailable": wl.no_reference}))
        return
    if hasattr(wl, "run_reference"):
        line = wl.run_reference(ref, args)
    else:
        ms = time_host_lib(wl, ref, max(1, min(args.steps, 5)), max(1, min(args.warmup, 2)))
        m = wl.metric(ms)
        line = dict(m)
        line.update({"ms_per_step": ms, "cpu_baseline": {"value": m["value"], "unit": m["unit"], "cores": REF_MT_CORES, "kind": "reference", "sample": "the full step, %s" % wl.name},
                     "config": {"workload": wl.name}, "dtype": args.dtype})
    line.update({"impl": "reference", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "scaling": "strong",
                 "vs_baseline": None, "data": "synthetic", "gpu_launches": 0,
                 "e2e": {"value": line["value"], "unit": line["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--config", default=os.environ.get("TRAINLIB_BENCH_CONFIG", "c5"))
    ap.add_argument("--dtype", default=None, choices=["fp32", "fp16"], help="default: fp32, fp16 for config 4")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-fusion", action="store_true", help="config 5: issue the reference's separate calls for norm, residual sum and ReLU instead of the fused extension calls")
    ap.add_argument("--no-graph", action="store_true", help="time the plain entry-point calls instead of a CUDA-graph replay (single-layer configs)")
    args = ap.parse_args()
    if args.dtype is None:
        args.dtype = "fp16" if args.config == "c4" else "fp32"
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    pkg = load_pkg()
    if args.impl == "reference":
        run_reference(args, pkg)
        return

    rank = int(os.environ.get("RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1")); local = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lib = pkg.load()
    rc = lib.trainlib_init(local)
    if rc != 0:
        raise SystemExit("trainlib_init failed: %s" % lib.trainlib_last_error_string().decode())
    wl = make_workload(args.config, pkg, lib, args.dtype)
    if hasattr(wl, "run"):
        line = wl.run(args, rank, world, dist)
    else:
        line = run_single(args, pkg, lib, wl)
    if rank == 0:
        print(json.dumps(line))
    if dist is not None:
        dist.barrier(); dist.destroy_process_group()


def run_single(args, pkg, lib, wl):
    pk = peaks()
    wl.setup_device()
    for _ in range(args.warmup):
        wl.step_device()
    lib.trainlib_synchronize(); pkg.check(lib)
    # the resident step is recorded once into a CUDA graph (the same entry-point calls, device pointers) and replayed:
    # at these sizes the calls are bound by launch latency, which the replay removes
    graph = None
    if getattr(wl, "use_graph", False) and not args.no_graph:
        lib.trainlib_graph_begin(); wl.step_device(); graph = lib.trainlib_graph_end()
        pkg.check(lib)
        for _ in range(2):
            lib.trainlib_graph_launch(graph)
        lib.trainlib_synchronize(); pkg.check(lib)
    sampler = ClockSampler(lib.trainlib_device()); sampler.start()
    launches0 = lib.trainlib_kernel_launches()
    ms = []
    for _ in range(args.steps):
        wl.l2_flush()
        lib.trainlib_timer_start()
        if graph:
            lib.trainlib_graph_launch(graph)
        else:
            wl.step_device()
        ms.append(lib.trainlib_timer_stop_ms())
    launches = lib.trainlib_kernel_launches() - launches0
    clocks = sampler.stop()
    pkg.check(lib)
    ms_step = float(np.mean(ms))
    # end to end through the C ABI with pinned host buffers (copies inside the timed region)
    e2e_ms = time_host_lib(wl, lib, args.steps, args.warmup)
    pkg.check(lib)
    m = wl.metric(ms_step); e = wl.metric(e2e_ms)
    line = {"metric": m["metric"], "value": m["value"], "unit": m["unit"], "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16" if args.dtype == "fp16" else "f32",
            "data": "synthetic", "config": {"workload": wl.name, "l2": "flushed between timed steps (256 MiB memset)",
                                            "replay": "CUDA graph of the entry-point calls of one step" if graph else "entry-point calls"},
            "roofline": wl.roofline(ms_step, pk), "gpu_launches": int(launches), "clocks": clocks,
            "e2e": {"value": e["value"], "unit": e["unit"], "h2d_bytes_per_step": int(wl.h2d), "d2h_bytes_per_step": int(wl.d2h), "ms_per_step": e2e_ms}}
    if not args.no_cpu_baseline and getattr(wl, "no_reference", None):
        line["cpu_baseline"] = {"value": None, "unit": m["unit"], "cores": 0, "kind": "reference", "sample": "none: " + wl.no_reference}
    elif not args.no_cpu_baseline and os.path.exists(REF_MT):
        ref = pkg.bind(ctypes.CDLL(REF_MT))
        wr = make_workload(args.config, pkg, ref, args.dtype)
        cms = time_host_lib(wr, ref, 3, 1)
        c = wr.metric(cms)
        line["cpu_baseline"] = {"value": c["value"], "unit": c["unit"], "cores": REF_MT_CORES, "kind": "reference", "sample": "3 full steps of %s" % wl.name, "ms_per_step": cms}
    return line


if __name__ == "__main__":
    main()
