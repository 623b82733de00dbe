#!/usr/bin/env python
"""Benchmark of the hot path on B200: the convolution stack of a benchmark network, or the GEMMs.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
                  [--net alexnet|vgg_a|gemm] [--scaling strong|weak]

alexnet (default) / vgg_a: one step = one forward + backward + weight-update pass over one
synthetic minibatch through the public API (NervanaGPU.fprop_conv / bprop_conv / update_conv /
fprop_pool / bprop_pool and the generated element-wise kernels for the ReLU mask and the SGD
step). With --gpus N > 1 (launched by torchrun, one rank per GPU) the minibatch of the
configuration (128 images for AlexNet, 64 for VGG model A) is split over the GPUs, N/g images
each (`--scaling strong`, the default: the split the configurations name), or every GPU runs a
whole minibatch of its own (`--scaling weak`); the fp32 weight gradients are summed over the GPUs
with NCCL all-reduces that overlap the backward pass.
gemm: `ng.dot` on the 2048^3 TN + ReLU product (the metric) and the fully-connected shapes.

Prints ONE JSON line (rank 0). `value` is device-timed with the inputs resident in HBM; `e2e`
repeats the measurement with the minibatch copied from pinned host memory and the last
activation read back every step. `--impl reference` times the reference's numpy validation path
(the oracle) of the same step on the host cores instead.
"""
import os
import sys

if "--impl" in sys.argv and "reference" in sys.argv:
    # The CPU arm uses every host core; launchers (torchrun) pin OMP_NUM_THREADS to 1 otherwise.
    # Must happen before numpy loads its BLAS.
    for _v in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        os.environ[_v] = str(os.cpu_count() or 1)

import argparse
import ctypes
import hashlib
import json
import subprocess
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

UNIT = "TFLOP/s"
METRICS = {
    "alexnet": ("alexnet_conv_stack_fprop_bprop_update_tflops", "BASELINE config 3"),
    "vgg_a": ("vgg_a_conv_stack_fprop_bprop_update_tflops", "BASELINE config 4"),
    "gemm": ("gemm_2048_tn_relu_tflops", "BASELINE config 1 (+ the shapes of config 2)"),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
JSON_OUT = sys.stdout


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--net", default="alexnet", choices=["alexnet", "vgg_a", "gemm"])
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-replay", action="store_true",
                    help="launch every kernel from Python instead of replaying a recorded step")
    return ap.parse_args()


# ---------------------------------------------------------------------------------------------
# host-side baseline: the oracle (numpy restatement of the reference's validation math) on the
# same step: every convolution's three passes, the max-pools, the ReLU masks and the SGD step
# ---------------------------------------------------------------------------------------------
class CpuStack(object):
    def __init__(self, net, seed=1003):
        from oracle import reference_math as rm
        self.rm = rm
        rm.keep_workspaces(True)      # the same shapes every step: allocate the big temporaries once
        rng = np.random.default_rng(seed)
        N, C, H, W = net["N"], net["C"], net["H"], net["W"]
        self.layers = []
        for kind, prm in net["layers"]:
            if kind == "conv":
                K, R, S, pad, stride = prm
                d = rm.ConvDims(N, C, K, 1, H, W, 1, R, S, 0, pad, pad, 1, stride, stride)
                w = rng.normal(0.0, 0.01, d.dimF).astype(np.float16).astype(np.float32)
                self.layers.append(["conv", d, w])
                C, (_, H, W) = K, d.MPQ
            else:
                R, S, stride = prm
                d = rm.PoolDims(N, C, 1, H, W, 1, 1, R, S, 0, 0, 0, 0, 1, 1, stride, stride)
                self.layers.append(["pool", d, None])
                _, H, W = d.MPQ
        first, last = self.layers[0][1], self.layers[-1][1]
        self.input = rng.uniform(0.0, 1.0, first.dimI).astype(np.float16).astype(np.float32)
        self.top = (rng.uniform(-1.0, 1.0, last.dimO) * 0.125).astype(np.float16).astype(np.float32)
        convs = [l[1] for l in self.layers if l[0] == "conv"]
        self.flops = 3 * sum(d.flops for d in convs) - convs[0].flops     # no input gradient for layer 1

    def step(self, lr=-1e-4):
        rm = self.rm
        x, acts = self.input, []
        for kind, d, w in self.layers:
            y = rm.conv_fprop_fast(d, x, w, relu=True) if kind == "conv" else rm.pool_max_fast(d, x)[0]
            y = y.astype(np.float16).astype(np.float32)
            acts.append(y)
            x = y
        grad = self.top
        for i in range(len(self.layers) - 1, -1, -1):
            kind, d, w = self.layers[i]
            x = self.input if i == 0 else acts[i - 1]
            if kind == "conv":
                grad = grad * (acts[i] > 0)                                   # Layer.bprop_relu
                dx = rm.conv_bprop_fast(d, w, grad).astype(np.float16).astype(np.float32) if i > 0 else None
                dw = rm.conv_update_fast(d, x, grad)
                self.layers[i][2] = (w + dw * np.float32(lr)).astype(np.float16).astype(np.float32)
            else:
                dx = rm.pool_max_fast(d, x, grad)[1].astype(np.float16).astype(np.float32)
            grad = dx


def host_threads():
    try:
        from threadpoolctl import threadpool_info
        n = max([p.get("num_threads", 1) for p in threadpool_info()] + [1])
        return int(n)
    except Exception:
        return os.cpu_count() or 1


def time_cpu(net, steps, warmup):
    stack = CpuStack(net)
    for _ in range(warmup):
        stack.step()
    t0 = time.perf_counter()
    for _ in range(steps):
        stack.step()
    dt = (time.perf_counter() - t0) / steps
    return stack.flops / dt / 1e12, dt * 1e3


def cpu_gemm(steps, warmup):
    from oracle import reference_math as rm
    rng = np.random.default_rng(1001)
    A = rng.standard_normal((2048, 2048)).astype(np.float16).astype(np.float32)
    B = rng.standard_normal((2048, 2048)).astype(np.float16).astype(np.float32)
    for _ in range(warmup):
        rm.gemm(A, B, a_t=True, relu=True)
    t0 = time.perf_counter()
    for _ in range(steps):
        rm.gemm(A, B, a_t=True, relu=True)
    dt = (time.perf_counter() - t0) / steps
    return 2.0 * 2048 ** 3 / dt / 1e12, dt * 1e3


def workload_text(args, net, per_gpu, world):
    metric, cfg = METRICS[args.net]
    if args.net == "gemm":
        return "ng.dot 2048x2048x2048, A stored k x m (TN), ReLU, fp16 round to nearest (%s)" % cfg
    split = ("minibatch of %d split over %d GPUs, %d images each" % (net["N"], world, per_gpu)
             if per_gpu != net["N"] else "minibatch of %d per GPU" % per_gpu)
    return ("%s, %s, fp16 CHWN, fprop+bprop+update, relu fused, max-pools, SGD step (%s)"
            % (net["name"], split, cfg))


def run_reference_arm(args, rank, world):
    if rank != 0:
        return
    from nervanagpu_b200.convnet import NETWORKS
    metric, _ = METRICS[args.net]
    cores = host_threads()
    if args.net == "gemm":
        tflops, ms = cpu_gemm(max(1, args.steps), max(0, args.warmup))
        net, sample = None, "the whole 2048^3 product per step (numpy fp32 sgemm + ReLU)"
    else:
        net = NETWORKS[args.net]
        tflops, ms = time_cpu(net, max(1, args.steps), max(0, args.warmup))
        sample = ("one whole step per step: every convolution's fprop / bprop / update, the max-pools, ReLU masks and "
                  "SGD of the %s minibatch of %d through the vectorised numpy oracle" % (net["name"], net["N"]))
    per_gpu = net["N"] // world if (net and args.scaling == "strong") else (net["N"] if net else 0)
    line = {
        "impl": "reference", "metric": metric, "value": tflops, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_text(args, net, per_gpu, world), "sample": sample},
        "cpu_baseline": {"value": tflops, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample,
                         "blas_threads_env": os.environ.get("OMP_NUM_THREADS")},
        "e2e": {"value": tflops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------
class ClockSampler(object):
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.samples = []
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(device), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), line.strip()))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass

    def summary(self, t0, t1):
        rows = []
        for ts, line in self.samples:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                rows.append((ts, float(parts[0]), float(parts[1]), parts[3:7]))
            except ValueError:
                continue
        inside = [r for r in rows if t0 <= r[0] <= t1] or rows[-3:]
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for r in inside for i in range(4) if r[3][i].lower().startswith("active")})
        return {"sm_mhz": float(np.median([r[1] for r in inside])), "sm_max_mhz": inside[0][2],
                "reasons": reasons, "samples": len(inside)}


# ---------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------
def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def pick_peak(peaks, clocks):
    """The burst figure applies while the SM clock stays at its maximum with no power cap (a short
    timed region), the sustained one otherwise. Returns (peak, name)."""
    burst = float(peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
    sustained = float(peaks.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops_sustained"]))
    at_max = (clocks and clocks.get("sm_mhz") and clocks.get("sm_max_mhz") and
              clocks["sm_mhz"] >= 0.97 * clocks["sm_max_mhz"] and "sw_power_cap" not in clocks.get("reasons", []))
    return (burst, "bf16_tflops (burst)", sustained) if at_max else (sustained, "bf16_tflops_sustained", burst)


def kernel_sources_hash():
    """sha256 over the CUDA sources of the library: a recorded ncu figure is only quoted while the
    kernels it was captured from are unchanged."""
    h = hashlib.sha256()
    csrc = os.path.join(ROOT, "nervanagpu_b200", "csrc")
    for name in sorted(os.listdir(csrc)):
        if name.endswith((".cu", ".cuh", ".h")):
            with open(os.path.join(csrc, name), "rb") as f:
                h.update(name.encode() + b"\0" + f.read())
    return h.hexdigest()


def recorded_traffic(key):
    """DRAM bytes (read + write) per launch of the dominant kernel from the ncu capture recorded in
    profiles/dram_traffic.json, or None when the kernels have changed since it was taken."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    try:
        with open(path) as f:
            rec = json.load(f)
        entry = rec[key]
        if entry.get("kernel_sources_sha256") != kernel_sources_hash():
            return None
        return entry["dram_bytes_per_launch"]
    except Exception:
        return None


class LaunchProbe(object):
    """Times every launch of one pass with its own CUDA event pair on the launching stream."""

    def __init__(self, ng):
        self.ng = ng
        self.events = []
        self.records = []

    def _pair(self, i):
        from nervanagpu_b200 import _lib
        while len(self.events) <= i:
            a, b = ctypes.c_void_p(), ctypes.c_void_p()
            _lib.check(self.ng.lib.ng_event_create(ctypes.byref(a)))
            _lib.check(self.ng.lib.ng_event_create(ctypes.byref(b)))
            self.events.append((a, b))
        return self.events[i]

    def begin_pass(self):
        self.calls = []

    def __call__(self, name, layer, launch):
        from nervanagpu_b200 import _lib
        a, b = self._pair(len(self.calls))
        _lib.check(self.ng.lib.ng_event_record(a, self.ng.stream))
        launch()
        _lib.check(self.ng.lib.ng_event_record(b, self.ng.stream))
        self.calls.append((name, layer))

    def end_pass(self):
        from nervanagpu_b200 import _lib
        self.ng.synchronize()
        for i, (name, layer) in enumerate(self.calls):
            ms = ctypes.c_float()
            a, b = self.events[i]
            _lib.check(self.ng.lib.ng_event_elapsed_ms(a, b, ctypes.byref(ms)))
            self.records.append((name, layer, ms.value))


class Ranks(object):
    """Rendezvous, barrier and reductions over the ranks (torch.distributed with gloo: plumbing)."""

    def __init__(self):
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist
            dist.init_process_group("gloo", rank=self.rank, world_size=self.world)
            self.dist = dist

    def _reduce(self, x, op):
        if self.dist is None:
            return x
        import torch
        t = torch.tensor([x], dtype=torch.float64)
        self.dist.all_reduce(t, op=getattr(self.dist.ReduceOp, op))
        return float(t[0])

    def max(self, x): return self._reduce(x, "MAX")
    def min(self, x): return self._reduce(x, "MIN")
    def sum(self, x): return self._reduce(x, "SUM")

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()

    def close(self):
        if self.dist is not None:
            self.dist.destroy_process_group()


def make_comm(lib, ranks):
    from nervanagpu_b200 import _lib
    if ranks.world == 1:
        return None
    nbytes = lib.ng_comm_unique_id_bytes()
    ident = ctypes.create_string_buffer(nbytes)
    if ranks.rank == 0:
        _lib.check(lib.ng_comm_unique_id(ident))
    box = [ident.raw]
    ranks.dist.broadcast_object_list(box, src=0)
    ident = ctypes.create_string_buffer(box[0], nbytes)
    comm = ctypes.c_void_p()
    _lib.check(lib.ng_comm_init(ctypes.byref(comm), ranks.world, ranks.rank, ident))
    return comm


def make_peer(lib, ranks):
    """The peer-memory group of the ranks (staging buffers mapped into one another over CUDA IPC),
    when NG_PEER_SUM=1 asks for it; None otherwise, or when it cannot be set up (the gradient sums
    then all go through NCCL). Off by default: measured equal to NCCL + SGD kernel within the run-to-run
    spread on 2 and 4 GPUs (single launches 22-23 us against 25-27 us, whole steps the same)."""
    from nervanagpu_b200 import _lib
    if ranks.world == 1 or os.environ.get("NG_PEER_SUM", "0") != "1":
        return None
    group = ctypes.c_void_p()
    handle = ctypes.create_string_buffer(lib.ng_peer_handle_bytes())
    ok = lib.ng_peer_create(ctypes.byref(group), ranks.world, ranks.rank, handle) == 0
    box = [None] * ranks.world
    ranks.dist.all_gather_object(box, handle.raw if ok else None)
    if any(h is None for h in box):
        return None
    ok = lib.ng_peer_connect(group, b"".join(box)) == 0
    flags = [None] * ranks.world
    ranks.dist.all_gather_object(flags, ok)
    if not all(flags):
        sys.stderr.write("peer-memory group not available: %s\n" % lib.ng_last_error().decode("utf-8", "replace"))
        return None
    return group


def counter(lib, fn):
    from nervanagpu_b200 import _lib
    c = ctypes.c_ulonglong()
    _lib.check(fn(ctypes.byref(c)))
    return c.value


def check_allreduce(stack, ranks):
    """One step's weight gradients, summed over the ranks by the library (NCCL), against the sum of
    the ranks' own gradients formed on the host side (gloo); and the weights after the step must
    be the same bits on every rank. Returns (sum is right, weights agree)."""
    ng = stack.ng
    comm, stack.comm = stack.comm, None
    w0 = stack.weights_flat.get()
    stack.fprop()
    lr, stack.lr = stack.lr, 0.0          # gradients only: leave the weights alone
    stack.bprop()
    ng.synchronize()
    local = stack.grads_flat.get().astype(np.float64)
    stack.lr, stack.comm = lr, comm
    import torch
    t = torch.from_numpy(local.copy())
    ranks.dist.all_reduce(t)              # sum over ranks, in double
    want = t.numpy()
    stack.weights_flat.set(w0)
    stack.lr = 0.0
    stack.step()                          # the same gradients, this time summed by the library
    ng.synchronize()
    stack.lr = lr
    got = stack.grads_flat.get().astype(np.float64)
    scale = np.abs(want).max() + 1e-30
    sum_ok = bool(np.abs(got - want).max() <= 1e-5 * scale * ranks.world)
    stack.weights_flat.set(w0)
    stack.step()
    ng.synchronize()
    w = stack.weights_flat.get().view(np.uint16).astype(np.float64)
    digest = float((w * (1 + np.arange(w.size) % 8191)).sum())
    same = ranks.max(digest) == ranks.min(digest)
    moved = bool((stack.weights_flat.get() != w0).any())
    return sum_ok, bool(same and moved)


def bench_gemm(args, ranks):
    from nervanagpu_b200 import NervanaGPU, _lib
    from nervanagpu_b200.convnet import StepTimer
    metric, cfg = METRICS["gemm"]
    ng = NervanaGPU(stochastic_round=False, bench=False, device=ranks.local_rank)
    lib = ng.lib
    ng.stream = ng.new_stream()
    timer = StepTimer(ng)
    rng = np.random.default_rng(1001)
    sampler = ClockSampler(ranks.local_rank) if ranks.rank == 0 else None

    def operands(op, m, n, k, std):
        A = rng.normal(0, std, (k, m) if op[0] == "t" else (m, k)).astype(np.float16)
        B = rng.normal(0, std, (n, k) if op[1] == "t" else (k, n)).astype(np.float16)
        return A, B

    # several operand sets, rotated, so that consecutive calls do not find their inputs in the L2
    def timed(op, m, n, k, relu, steps, std=1.0, sets=None):
        nbytes = 2 * (m * k + k * n + m * n)
        sets = sets or max(2, int(np.ceil(300e6 / nbytes)))
        ops = []
        for _ in range(sets):
            A, B = operands(op, m, n, k, std)
            dA, dB = ng.array(A), ng.array(B)
            ops.append((dA.T if op[0] == "t" else dA, dB.T if op[1] == "t" else dB, ng.empty((m, n))))
        i = [0]

        def call():
            a, b, c = ops[i[0] % sets]
            i[0] += 1
            ng.dot(a, b, c, relu=relu)
        for _ in range(max(args.warmup, 3)):
            call()
        ng.synchronize()
        ms = timer.time_ms(call, steps) / steps
        return ms, 2.0 * m * n * k / (ms * 1e-3) / 1e12, nbytes / (ms * 1e-3) / 1e9, sets

    ranks.barrier()
    l0 = counter(lib, lib.ng_launch_count)
    t0 = time.time()
    ms, tflops, _, sets = timed("tn", 2048, 2048, 2048, True, args.steps)
    ng.synchronize()
    t1 = time.time()
    launches = counter(lib, lib.ng_launch_count) - l0 - max(args.warmup, 3)
    ms = ranks.max(ms)
    tflops = 2.0 * 2048 ** 3 / (ms * 1e-3) / 1e12

    # end to end: operands from pinned host memory every call, result read back
    A, B = operands("tn", 2048, 2048, 2048, 1.0)
    nb = A.nbytes
    pins = []
    for src in (A, B):
        p = ctypes.c_void_p()
        _lib.check(lib.ng_host_alloc(ctypes.byref(p), nb))
        ctypes.memmove(p.value, src.ctypes.data, nb)
        pins.append(p)
    pin_c = ctypes.c_void_p()
    _lib.check(lib.ng_host_alloc(ctypes.byref(pin_c), nb))
    dA, dB, dC = ng.empty((2048, 2048)), ng.empty((2048, 2048)), ng.empty((2048, 2048))

    def e2e_call():
        _lib.check(lib.ng_memcpy_h2d_async(dA.ptr, pins[0], nb, ng.stream))
        _lib.check(lib.ng_memcpy_h2d_async(dB.ptr, pins[1], nb, ng.stream))
        ng.dot(dA.T, dB, dC, relu=True)
        _lib.check(lib.ng_memcpy_d2h_async(pin_c, dC.ptr, nb, ng.stream))
    for _ in range(3):
        e2e_call()
    ng.synchronize()
    w0 = time.perf_counter()
    e2e_dev = timer.time_ms(e2e_call, args.steps)
    ng.synchronize()
    e2e_ms = ranks.max(max(e2e_dev, (time.perf_counter() - w0) * 1e3)) / args.steps
    if sampler is not None:
        sampler.stop()

    others = {}
    for name, (op, m, n, k) in {"3072_nn": ("nn", 3072, 3072, 3072), "3072_nt": ("nt", 3072, 3072, 3072),
                                "3072_tn": ("tn", 3072, 3072, 3072), "fc_4096x128x9216": ("nn", 4096, 128, 9216),
                                "fc_4096x128x4096": ("nn", 4096, 128, 4096), "fc_1000x128x4096": ("nn", 1000, 128, 4096),
                                "fc_9216x4096x128": ("nn", 9216, 4096, 128)}.items():
        o_ms, o_tf, o_gbs, _ = timed(op, m, n, k, False, min(args.steps, 50), std=0.1)
        others[name] = {"us": o_ms * 1e3, "tflops": o_tf, "gbs": o_gbs}
    if ranks.rank != 0:
        return
    clocks = sampler.summary(t0, t1) if sampler is not None else None
    peaks, peak_src = load_peaks()
    peak, peak_name, other_peak = pick_peak(peaks, clocks)
    line = {
        "metric": metric, "value": tflops * ranks.world, "unit": UNIT, "n_gpus": ranks.world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": workload_text(args, None, 0, ranks.world),
                   "l2": "%d operand sets rotated (%d MB): consecutive calls read operands that left the L2"
                         % (sets, sets * 25),
                   "other_shapes": others},
        "e2e": {"value": 2.0 * 2048 ** 3 / (e2e_ms * 1e-3) / 1e12 * ranks.world, "unit": UNIT,
                "h2d_bytes_per_step": 2 * nb, "d2h_bytes_per_step": nb, "ms_per_step": e2e_ms},
        "gpu_launches": int(launches), "clocks": clocks,
        "roofline": {"bound": "tensor", "achieved": tflops, "peak": peak, "unit": "TFLOP/s", "frac": tflops / peak,
                     "frac_of_other_peak": tflops / other_peak, "peak_source": "%s %s" % (peak_src, peak_name),
                     "traffic": recorded_traffic("gemm_2048_tn"), "kernel": "igemm_tc_kernel<gemm>"},
        "fallback_launches": int(counter(lib, lib.ng_fallback_launch_count)),
    }
    if ranks.world == 1 and not args.no_cpu_baseline:
        c_tf, _ = cpu_gemm(5, 1)
        line["cpu_baseline"] = {"value": c_tf, "unit": UNIT, "cores": host_threads(), "kind": "port",
                                "sample": "the whole 2048^3 product (numpy fp32 sgemm + ReLU), 5 repeats"}
    JSON_OUT.write(json.dumps(line) + "\n")
    JSON_OUT.flush()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args, int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")))
        return

    # Keep stdout to the one JSON line: the line is written to a private copy of the original
    # stdout, and file descriptor 1 is pointed at stderr for everything else (NCCL prints its
    # version banner on stdout from C).
    sys.stdout.flush()
    global JSON_OUT
    JSON_OUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    ranks = Ranks()
    rank, world = ranks.rank, ranks.world
    if args.net == "gemm":
        bench_gemm(args, ranks)
        ranks.close()
        return

    from nervanagpu_b200 import NervanaGPU, _lib
    from nervanagpu_b200.convnet import ConvStack, NETWORKS, StepTimer

    ng = NervanaGPU(stochastic_round=False, bench=False, device=ranks.local_rank)
    lib = ng.lib
    ng.stream = ng.new_stream()      # a stream of its own: recorded sequences cannot use the default one
    comm = make_comm(lib, ranks)

    net = NETWORKS[args.net]
    metric, cfg_name = METRICS[args.net]
    strong = args.scaling == "strong"
    if strong:
        stack = ConvStack(ng, net, seed=1003, comm=comm, shard=(rank, world))
    else:
        stack = ConvStack(ng, net, seed=1003, data_seed=2003 + rank, comm=comm)
    if os.environ.get("NG_BUCKET_FRACTION"):     # measurement aid: where the first gradient bucket ends
        from nervanagpu_b200.convnet import comm_bucket_order
        stack.comm_buckets = comm_bucket_order([l.sizeF for l in stack.convs], float(os.environ["NG_BUCKET_FRACTION"]))
    stack.peer = make_peer(lib, ranks)
    stack.peer_max_bytes = lib.ng_peer_max_bytes() if stack.peer is not None else 0
    timer = StepTimer(ng)

    def barrier():
        ng.synchronize()
        ranks.barrier()

    sampler = ClockSampler(ranks.local_rank) if rank == 0 else None

    # ---- one live step: which kernels serve it ---------------------------------------------
    f0 = counter(lib, lib.ng_fallback_launch_count)
    stack.step()
    ng.synchronize()
    fallback = counter(lib, lib.ng_fallback_launch_count) - f0
    allreduce_ok = weights_in_step = None
    if world > 1:
        allreduce_ok, weights_in_step = check_allreduce(stack, ranks)

    # ---- device-resident measurement ------------------------------------------------------
    # The step is recorded once per input buffer and replayed (one host call per step instead of
    # ~33 launches); with several GPUs the NCCL all-reduces are part of the recording.
    def prepare(with_replay):
        for _ in range(max(args.warmup, 3)):
            stack.step()
        stack._recorded = None
        fn = stack.step
        if with_replay:
            ok = 1
            try:
                stack.record_steps()
            except _lib.NervanaError as exc:
                sys.stderr.write("recording the step failed (%s): launching kernel by kernel\n" % exc)
                ok = 0
            with_replay = ranks.min(ok) == 1      # every rank must take the same route
            if not with_replay:
                stack._recorded = None
        if with_replay:
            fn = stack.step_prefetched            # nothing prefetched yet: replays on the resident input
            # the replayed form gets its warm-up too: the first replays of a recording upload it and,
            # with several GPUs, let NCCL finish setting up its recorded collectives
            for _ in range(max(args.warmup, 3)):
                fn()
            ng.synchronize()
        return fn, with_replay

    def timed_steps(fn):
        barrier()
        ms = timer.time_ms(fn, args.steps)
        ng.synchronize()
        barrier()
        return ranks.max(ms) / args.steps

    step_fn, replay = prepare(not args.no_replay)
    l0 = counter(lib, lib.ng_launch_count)
    t0 = time.time()
    ms_step = timed_steps(step_fn)
    t1 = time.time()
    gpu_launches = counter(lib, lib.ng_launch_count) - l0
    units = stack.flops * world              # flops of all ranks per step (strong: one minibatch)
    value = units / (ms_step * 1e-3) / 1e12

    # the same step without the gradient exchange: what the all-reduces add to the step
    exposed_comm_ms = None
    if world > 1:
        stack.comm = None
        fn_nc, _ = prepare(replay)
        exposed_comm_ms = ms_step - timed_steps(fn_nc)
        stack.comm = comm
        step_fn, replay = prepare(replay)

    # ---- end to end: pinned host minibatch in, last activation out, every step ---------------
    in_bytes = stack.input.nbytes
    out_t = stack.acts[-1]
    out_bytes = out_t.nbytes
    pin_in, pin_out = ctypes.c_void_p(), ctypes.c_void_p()
    _lib.check(lib.ng_host_alloc(ctypes.byref(pin_in), in_bytes))
    _lib.check(lib.ng_host_alloc(ctypes.byref(pin_out), out_bytes))
    ctypes.memmove(pin_in.value, stack.host_input.ctypes.data, in_bytes)

    # Every step copies its own minibatch from pinned host memory and returns its last activation
    # to the host. Both copies are pipelined, as a training loop does it: the copy of minibatch i+1
    # runs on a second stream while step i computes (ConvStack.prefetch_input / step_prefetched),
    # the result of step i is read back on a third stream while step i+1 computes, and the host
    # takes delivery of it (waits for that copy) one step later. The host is never more than one
    # step ahead of the device, and all K reads have completed when the timed region ends.
    pin_out_b = ctypes.c_void_p()
    _lib.check(lib.ng_host_alloc(ctypes.byref(pin_out_b), out_bytes))
    pin_outs = [pin_out, pin_out_b]
    read_stream = ng.new_stream()
    ev_step = ctypes.c_void_p()
    _lib.check(lib.ng_event_create(ctypes.byref(ev_step)))
    ev_read = [ctypes.c_void_p(), ctypes.c_void_p()]
    for ev in ev_read:
        _lib.check(lib.ng_event_create(ctypes.byref(ev)))
    e2e_count = [0]

    stage = [ng.empty(out_t.shape, dtype=np.float16), ng.empty(out_t.shape, dtype=np.float16)]

    def e2e_step():
        i = e2e_count[0]
        stack.step_prefetched()                      # waits (on the device) for its minibatch
        stack.prefetch_input(pin_in)                 # next minibatch, overlapped with this step
        # the result leaves through one of two device staging buffers, so that the next step
        # (which overwrites the activation) does not have to wait for the copy to the host
        if i > 1:
            _lib.check(lib.ng_stream_wait_event(ng.stream, ev_read[i % 2]))   # read of step i-2: long done
        _lib.check(lib.ng_memcpy_d2d_async(stage[i % 2].ptr, out_t.ptr, out_bytes, ng.stream))
        _lib.check(lib.ng_event_record(ev_step, ng.stream))
        _lib.check(lib.ng_stream_wait_event(read_stream, ev_step))
        _lib.check(lib.ng_memcpy_d2h_async(pin_outs[i % 2], stage[i % 2].ptr, out_bytes, read_stream))
        _lib.check(lib.ng_event_record(ev_read[i % 2], read_stream))
        if i > 0:     # delivery of the previous step's result
            _lib.check(lib.ng_event_sync(ev_read[(i - 1) % 2]))
        e2e_count[0] = i + 1

    stack.prefetch_input(pin_in)
    for _ in range(3):
        e2e_step()
    barrier()
    w0 = time.perf_counter()
    e2e_ms_dev = timer.time_ms(e2e_step, args.steps)
    ng.synchronize()                                 # includes the last prefetch: K steps, K copies
    e2e_wall = (time.perf_counter() - w0) * 1e3
    barrier()
    e2e_ms = ranks.max(max(e2e_ms_dev, e2e_wall)) / args.steps
    e2e_value = units / (e2e_ms * 1e-3) / 1e12
    if sampler is not None:
        sampler.stop()

    # ---- per-launch timing of the tensor-core engine (roofline) --------------------------------
    # (launch by launch on one stream: the weight updates do not overlap the backward chain here, so
    # the sum of this breakdown is larger than the step time above)
    stack._recorded = None
    stack.overlap_update = False
    stack.step()                      # sizes the main stream's scratch memory outside the timed passes
    ng.synchronize()
    probe = LaunchProbe(ng)
    stack.probe = probe
    for _ in range(5):
        probe.begin_pass()
        stack.step()
        probe.end_pass()
    stack.probe = None
    conv_ms = conv_flops = 0.0
    per_kind = {}
    for name, layer, ms in probe.records:
        per_kind.setdefault(name, [0.0, 0])
        per_kind[name][0] += ms
        per_kind[name][1] += 1
        if name in ("fprop_conv", "bprop_conv", "update_conv"):
            conv_ms += ms
            conv_flops += layer.flops
    n_conv = sum(per_kind[k][1] for k in ("fprop_conv", "bprop_conv", "update_conv"))
    achieved = conv_flops / (conv_ms * 1e-3) / 1e12 if conv_ms > 0 else 0.0
    barrier()

    if rank != 0:
        ranks.close()
        return

    clocks = sampler.summary(t0, t1) if sampler is not None else None
    peaks, peak_src = load_peaks()
    peak, peak_name, other_peak = pick_peak(peaks, clocks)
    line = {
        "metric": metric, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": args.scaling if world > 1 else "strong",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": workload_text(args, net, stack.N, world),
                   "global_batch": stack.N * world, "parallelism": "dp%d" % world,
                   "gflop_per_step_per_gpu": stack.flops / 1e9,
                   "l2": "no flush: activations+deltas of one step (~%d MB per GPU) %s the 126 MB L2"
                         % (int(sum(a.nbytes for a in stack.acts) * 2 / 1e6),
                            "exceed" if sum(a.nbytes for a in stack.acts) * 2 > 126e6 else "DO NOT exceed"),
                   "launch": "recorded step replayed (CUDA graph)" if replay else "one call per kernel"},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": in_bytes * world,
                "d2h_bytes_per_step": out_bytes * world, "ms_per_step": e2e_ms,
                "h2d_gbs_all_gpus": in_bytes * world / (e2e_ms * 1e-3) / 1e9,
                "launch": "recorded step replayed" if replay else "one call per kernel"},
        "gpu_launches": int(gpu_launches),
        "fallback_launches_per_step": int(fallback),
        "clocks": clocks,
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                     "frac": achieved / peak if peak else None,
                     "frac_of_other_peak": achieved / other_peak if other_peak else None,
                     "traffic": recorded_traffic("%s_step_n%d" % (args.net, stack.N)),
                     "traffic_unit": "bytes of DRAM read+write per conv launch (ncu, mean over the launches of a step)",
                     "peak_source": "%s %s" % (peak_src, peak_name),
                     "kernel": "igemm_tc_kernel (+ its split-K reduction / im2col satellites)",
                     "launches_timed": n_conv, "avg_launch_ms": conv_ms / n_conv if n_conv else None},
        "breakdown_ms_per_step": {k: v[0] / 5.0 for k, v in sorted(per_kind.items())},
    }
    if world > 1:
        line["allreduce_ok"] = allreduce_ok
        line["gradient_sum"] = ("NCCL all-reduce for the first bucket, peer-memory sum fused with the SGD step for "
                                "the later, small ones" if stack.peer is not None else "NCCL all-reduce, every bucket")
        line["weights_identical_across_ranks"] = weights_in_step
        line["allreduce_exposed_ms_per_step"] = exposed_comm_ms
    if world == 1 and not args.no_cpu_baseline:
        tflops, cpu_ms = time_cpu(net, 1, 1)
        line["cpu_baseline"] = {"value": tflops, "unit": UNIT, "cores": host_threads(), "kind": "port",
                                "sample": "one whole step of the same stack through the numpy oracle (%.0f ms)" % cpu_ms}
    JSON_OUT.write(json.dumps(line) + "\n")
    JSON_OUT.flush()
    ranks.close()


if __name__ == "__main__":
    main()
