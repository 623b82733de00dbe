#!/usr/bin/env python
"""Benchmark of the hot path: the AlexNet convolution stack (BASELINE config 3) on B200.

One step = one forward + backward + weight-update pass over one synthetic minibatch through the
public API (NervanaGPU.fprop_conv / bprop_conv / update_conv / fprop_pool / bprop_pool and the
generated element-wise kernels for the ReLU mask and the SGD step), N = 128 images per GPU.
With --gpus N > 1 (launched by torchrun, one rank per GPU) every rank runs the same per-GPU
minibatch (weak scaling) and the fp32 weight gradients are summed with one NCCL all-reduce.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--net alexnet|vgg_a]

Prints ONE JSON line (rank 0). `value` is device-timed with the inputs resident in HBM; `e2e`
repeats the measurement with the minibatch copied from pinned host memory and the last
activation read back every step. `--impl reference` times the reference's numpy validation path
(the oracle) on the host cores instead.
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

METRIC = "alexnet_conv_stack_fprop_bprop_update_tflops"
UNIT = "TFLOP/s"
# dram__bytes_read.sum + dram__bytes_write.sum per igemm_tc_kernel launch, from the ncu capture summarised
# in profiles/igemm_tc_kernel_alexnet_step_traffic.md (not measurable from inside this script)
TRAFFIC_BYTES_PER_CONV_LAUNCH = {("alexnet", 128): 27.92e6}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--net", default="alexnet", choices=["alexnet", "vgg_a"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-replay", action="store_true",
                    help="end-to-end arm launches every kernel from Python instead of replaying a recorded step")
    return ap.parse_args()


# ---------------------------------------------------------------------------------------------
# host-side baseline: the oracle (numpy restatement of the reference's validation math)
# ---------------------------------------------------------------------------------------------
CPU_SAMPLE = ("AlexNet conv3 (N=128, 192->384, 13x13, 3x3 pad 1) fprop+bprop+update through the vectorised "
              "numpy oracle (im2col + BLAS sgemm), one pass per step")


def cpu_sample_setup():
    from oracle import reference_math as rm
    cd = rm.ConvDims(128, 192, 384, 1, 13, 13, 1, 3, 3, 0, 1, 1, 1, 1, 1)
    rng = np.random.default_rng(1003)
    I = rng.uniform(0, 1, cd.dimI).astype(np.float16).astype(np.float32)
    F = rng.normal(0, 0.01, cd.dimF).astype(np.float16).astype(np.float32)
    E = (rng.uniform(-1, 1, cd.dimO) * 0.125).astype(np.float16).astype(np.float32)

    def one_pass():
        rm.conv_fprop_fast(cd, I, F, relu=True)
        rm.conv_bprop_fast(cd, F, E)
        rm.conv_update_fast(cd, I, E)
    return one_pass, 3 * cd.flops


def host_threads():
    try:
        from threadpoolctl import threadpool_info
        n = max([p.get("num_threads", 1) for p in threadpool_info()] + [1])
        return int(n)
    except Exception:
        return os.cpu_count() or 1


def time_cpu(steps, warmup):
    one_pass, flops = cpu_sample_setup()
    for _ in range(warmup):
        one_pass()
    t0 = time.perf_counter()
    for _ in range(steps):
        one_pass()
    dt = (time.perf_counter() - t0) / steps
    return flops / dt / 1e12, dt * 1e3


def run_reference_arm(args, rank):
    if rank != 0:
        return
    tflops, ms = time_cpu(max(1, args.steps), max(0, args.warmup))
    cores = host_threads()
    line = {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "alexnet conv stack N=128 fprop+bprop+update (BASELINE config 3)",
                   "sample": CPU_SAMPLE},
        "cpu_baseline": {"value": tflops, "unit": UNIT, "cores": cores, "kind": "port", "sample": CPU_SAMPLE},
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


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference_arm(args, rank)
        return

    # keep stdout to the one JSON line: NCCL's version banner goes to stderr
    os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
    dist = None
    if world > 1:
        import torch.distributed as dist   # plumbing only: rendezvous, barrier, max over ranks
        dist.init_process_group("gloo", rank=rank, world_size=world)

    from nervanagpu_b200 import NervanaGPU, _lib
    from nervanagpu_b200.convnet import ConvStack, NETWORKS, StepTimer

    ng = NervanaGPU(stochastic_round=False, bench=False, device=local_rank)
    lib = ng.lib
    ng.stream = ng.new_stream()      # a stream of its own: recorded sequences cannot use the default one

    comm = None
    if world > 1:
        nbytes = lib.ng_comm_unique_id_bytes()
        ident = ctypes.create_string_buffer(nbytes)
        if rank == 0:
            _lib.check(lib.ng_comm_unique_id(ident))
        box = [ident.raw]
        dist.broadcast_object_list(box, src=0)
        ident = ctypes.create_string_buffer(box[0], nbytes)
        comm = ctypes.c_void_p()
        _lib.check(lib.ng_comm_init(ctypes.byref(comm), world, rank, ident))

    net = NETWORKS[args.net]
    stack = ConvStack(ng, net, seed=1003 + rank, comm=comm)
    timer = StepTimer(ng)

    def barrier():
        ng.synchronize()
        if dist is not None:
            dist.barrier()

    def max_over_ranks(x):
        if dist is None:
            return x
        import torch
        t = torch.tensor([x], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    def min_over_ranks(x):
        if dist is None:
            return x
        import torch
        t = torch.tensor([x], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return float(t[0])

    def launches():
        c = ctypes.c_ulonglong()
        _lib.check(lib.ng_launch_count(ctypes.byref(c)))
        return c.value

    sampler = ClockSampler(local_rank) if rank == 0 else None

    # ---- device-resident measurement ------------------------------------------------------
    # The step is recorded once per input buffer and replayed (one host call per step instead of
    # ~33 launches); with several GPUs the per-layer NCCL all-reduces are part of the recording.
    replay = not args.no_replay
    for _ in range(max(args.warmup, 3)):
        stack.step()
    step_fn = stack.step
    if replay:
        ok = 1
        try:
            stack.record_steps()
        except _lib.NervanaError as exc:
            sys.stderr.write("recording the step failed (%s): launching kernel by kernel\n" % exc)
            ok = 0
        # every rank must take the same route
        replay = min_over_ranks(ok) == 1
        if not replay:
            stack._recorded = None
    if replay:
        step_fn = stack.step_prefetched          # nothing prefetched yet: replays on the resident input
        step_fn()
    barrier()
    l0 = launches()
    t0 = time.time()
    ms_total = timer.time_ms(step_fn, args.steps)
    ng.synchronize()
    t1 = time.time()
    gpu_launches = launches() - l0
    barrier()
    ms_total = max_over_ranks(ms_total)
    ms_step = ms_total / args.steps
    value = world * stack.flops / (ms_step * 1e-3) / 1e12

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
    e2e_ms = max_over_ranks(max(e2e_ms_dev, e2e_wall)) / args.steps
    e2e_value = world * stack.flops / (e2e_ms * 1e-3) / 1e12
    if sampler is not None:
        sampler.stop()

    # ---- per-launch timing of the tensor-core engine (roofline) --------------------------------
    # (launch by launch on one stream: the weight updates do not overlap the backward chain here, so
    # the sum of this breakdown is larger than the step time above)
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
    peaks, peak_src = load_peaks()
    peak = float(peaks.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops_sustained"]))
    achieved = conv_flops / (conv_ms * 1e-3) / 1e12 if conv_ms > 0 else 0.0

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    clocks = sampler.summary(t0, t1) if sampler is not None else None
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "%s N=%d per GPU, fp16 CHWN, fprop+bprop+update, relu fused, max-pools, SGD step "
                               "(BASELINE config 3)" % (net["name"], stack.N),
                   "global_batch": stack.N * world, "parallelism": "dp%d" % world,
                   "gflop_per_step_per_gpu": stack.flops / 1e9,
                   "l2": "no flush: activations+deltas of one step (~%d MB) exceed the 126 MB L2"
                         % int(sum(a.nbytes for a in stack.acts) * 2 / 1e6),
                   "launch": "recorded step replayed (CUDA graph)" if replay else "one call per kernel"},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": in_bytes, "d2h_bytes_per_step": out_bytes,
                "ms_per_step": e2e_ms, "launch": "recorded step replayed" if replay else "one call per kernel"},
        "gpu_launches": int(gpu_launches),
        "clocks": clocks,
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                     "frac": achieved / peak if peak else None,
                     "traffic": TRAFFIC_BYTES_PER_CONV_LAUNCH.get((args.net, stack.N)),
                     "traffic_unit": "bytes of DRAM read+write per conv launch (ncu, mean of the 14 launches of a step)",
                     "peak_source": "%s bf16_tflops_sustained" % peak_src,
                     "kernel": "igemm_tc_kernel (+ its split-K reduction / im2col satellites)",
                     "launches_timed": n_conv, "avg_launch_ms": conv_ms / n_conv if n_conv else None},
        "breakdown_ms_per_step": {k: v[0] / 5.0 for k, v in sorted(per_kind.items())},
    }
    if world == 1 and not args.no_cpu_baseline:
        tflops, _ = time_cpu(2, 1)
        line["cpu_baseline"] = {"value": tflops, "unit": UNIT, "cores": host_threads(), "kind": "port",
                                "sample": CPU_SAMPLE}
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
