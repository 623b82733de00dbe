"""Small stand-alone workloads for profiling single kernels (ncu) or timing single calls.

    python benchmarks/profile_cases.py <case> [--reps R] [--warm W]

A case is a name from the tables below plus, for convolutions, the pass ("vgg4_fprop"), or a
convolution spelled out: "conv:N,C,K,D,H,W,T,R,S,pad_d,pad_h,pad_w,str_d,str_h,str_w:fprop";
"step:alexnet:128" (or vgg_a, any minibatch) runs whole steps of the benchmark stack.

Each case allocates its operands once (tensors larger than the 126 MB L2 in total, a few
hundred MB at most), runs `warm` untimed calls, then `reps` calls timed with CUDA events, and
prints one JSON line with the time per call, the algorithmic work and the achieved rate.
"""
import argparse
import ctypes
import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from nervanagpu_b200 import NervanaGPU, _lib   # noqa: E402

CONV = {
    # name: (N, C, K, D, H, W, T, R, S, pad_d, pad_h, pad_w, str_d, str_h, str_w)
    "alex1": (128, 3, 64, 1, 224, 224, 1, 11, 11, 0, 2, 2, 1, 4, 4),
    # conv1 after a 4x4 space-to-depth of its input: 48 channels, 3x3, stride 1 (same flops as alex1 up to padding)
    "alex1_s2d": (128, 48, 64, 1, 57, 57, 1, 3, 3, 0, 0, 0, 1, 1, 1),
    "alex2": (128, 64, 192, 1, 27, 27, 1, 5, 5, 0, 2, 2, 1, 1, 1),
    "alex3": (128, 192, 384, 1, 13, 13, 1, 3, 3, 0, 1, 1, 1, 1, 1),
    "alex4": (128, 384, 256, 1, 13, 13, 1, 3, 3, 0, 1, 1, 1, 1, 1),
    "alex5": (128, 256, 256, 1, 13, 13, 1, 3, 3, 0, 1, 1, 1, 1, 1),
    "vgg1": (64, 3, 64, 1, 224, 224, 1, 3, 3, 0, 1, 1, 1, 1, 1),
    "vgg2": (64, 64, 128, 1, 112, 112, 1, 3, 3, 0, 1, 1, 1, 1, 1),
    "vgg3": (64, 128, 256, 1, 56, 56, 1, 3, 3, 0, 1, 1, 1, 1, 1),
    "vgg4": (64, 256, 256, 1, 56, 56, 1, 3, 3, 0, 1, 1, 1, 1, 1),
    "vgg5": (64, 256, 512, 1, 28, 28, 1, 3, 3, 0, 1, 1, 1, 1, 1),
    "vgg6": (64, 512, 512, 1, 28, 28, 1, 3, 3, 0, 1, 1, 1, 1, 1),
    "vgg7": (64, 512, 512, 1, 14, 14, 1, 3, 3, 0, 1, 1, 1, 1, 1),
    "c3d": (32, 64, 64, 16, 56, 56, 3, 3, 3, 1, 1, 1, 1, 1, 1),
}
POOL = {
    # name: (N, C, D, H, W, J, T, R, S, pad_j, pad_d, pad_h, pad_w, str_j, str_d, str_h, str_w)
    "alexpool1": (128, 64, 1, 55, 55, 1, 1, 3, 3, 0, 0, 0, 0, 1, 1, 2, 2),
    "alexpool2": (128, 192, 1, 27, 27, 1, 1, 3, 3, 0, 0, 0, 0, 1, 1, 2, 2),
    "alexpool3": (128, 256, 1, 13, 13, 1, 1, 3, 3, 0, 0, 0, 0, 1, 1, 2, 2),
    "vggpool1": (64, 64, 1, 224, 224, 1, 1, 2, 2, 0, 0, 0, 0, 1, 1, 2, 2),
    "pool4d": (32, 64, 16, 56, 56, 2, 2, 2, 2, 0, 0, 0, 0, 2, 2, 2, 2),
}
GEMM = {
    # name: (op, m, n, k)
    "gemm2048_tn": ("tn", 2048, 2048, 2048),
    "gemm3072_nn": ("nn", 3072, 3072, 3072),
    "gemm3072_nt": ("nt", 3072, 3072, 3072),
    "gemm3072_tn": ("tn", 3072, 3072, 3072),
    "fc_4096x128x9216_nn": ("nn", 4096, 128, 9216),
    "fc_4096x128x4096_nn": ("nn", 4096, 128, 4096),
    "fc_1000x128x4096_nn": ("nn", 1000, 128, 4096),
    "fc_9216x4096x128_nn": ("nn", 9216, 4096, 128),
    "gemm8192_nt": ("nt", 8192, 8192, 8192),
}


def _timed(ng, fn, warm, reps):
    lib = ng.lib
    a, b = ctypes.c_void_p(), ctypes.c_void_p()
    _lib.check(lib.ng_event_create(ctypes.byref(a)))
    _lib.check(lib.ng_event_create(ctypes.byref(b)))
    for _ in range(warm):
        fn()
    _lib.check(lib.ng_event_record(a, ng.stream))
    for _ in range(reps):
        fn()
    _lib.check(lib.ng_event_record(b, ng.stream))
    _lib.check(lib.ng_event_sync(b))
    ms = ctypes.c_float()
    _lib.check(lib.ng_event_elapsed_ms(a, b, ctypes.byref(ms)))
    ng.synchronize()
    return ms.value / reps


def _fill(ng, shape, dtype=np.float16, seed=0, lo=-1.0, hi=1.0):
    rng = np.random.default_rng(seed)
    t = ng.empty(shape, dtype=dtype)
    # generate in slabs to keep host memory small
    flat = t.reshape(int(np.prod(shape)))
    host = rng.uniform(lo, hi, min(flat.size, 1 << 22)).astype(dtype)
    pos = 0
    while pos < flat.size:
        n = min(host.size, flat.size - pos)
        flat[pos:pos + n].set(host[:n])
        pos += n
    return t


def run_case(name, warm=3, reps=10, sr=False):
    ng = NervanaGPU(stochastic_round=sr)
    if name.startswith("conv:") or ("_" in name and name.rsplit("_", 1)[0] in CONV and
                                    name.rsplit("_", 1)[1] in ("fprop", "bprop", "update")):
        if name.startswith("conv:"):
            _, dims, op = name.split(":")
            cfg = tuple(int(v) for v in dims.split(","))
        else:
            layer_name, op = name.rsplit("_", 1)
            cfg = CONV[layer_name]
        layer = ng.conv_layer(np.float16, *cfg)
        I = _fill(ng, layer.dimI, seed=1, lo=0.0)
        F = _fill(ng, layer.dimF, seed=2, lo=-0.02, hi=0.02)
        E = _fill(ng, layer.dimO, seed=3, lo=-0.125, hi=0.125)
        if op == "fprop":
            O = ng.empty(layer.dimO)
            fn = lambda: ng.fprop_conv(layer, I, F, O, relu=True)
        elif op == "bprop":
            gI = ng.empty(layer.dimI)
            fn = lambda: ng.bprop_conv(layer, F, E, gI)
        else:
            gF = ng.empty(layer.dimF, dtype=np.float32)
            fn = lambda: ng.update_conv(layer, I, E, gF)
        work, unit = layer.flops, "TFLOP/s"
        algo_bytes = 2 * (layer.sizeI + layer.sizeF + layer.sizeO) + (2 * layer.sizeF if op == "update" else 0)
    elif "_" in name and name.split("_")[0] in POOL:
        layer_name, op = name.split("_")[:2]
        cfg = POOL[layer_name]
        layer = ng.pool_layer(np.float16, "max", *cfg)
        I = _fill(ng, layer.dimI, seed=1, lo=0.0)
        if op == "fprop":
            O = ng.empty(layer.dimO)
            fn = lambda: ng.fprop_pool(layer, I, O)
            algo_bytes = 2 * (layer.sizeI + layer.sizeO)
        else:
            E = _fill(ng, layer.dimO, seed=3)
            gI = ng.empty(layer.dimI)
            fn = lambda: ng.bprop_pool(layer, I, E, gI)
            algo_bytes = 2 * (2 * layer.sizeI + layer.sizeO)
        work, unit = algo_bytes, "GB/s"
    elif name in GEMM:
        op, m, n, k = GEMM[name]
        A = _fill(ng, (k, m) if op[0] == "t" else (m, k), seed=1, lo=-0.2, hi=0.2)
        B = _fill(ng, (n, k) if op[1] == "t" else (k, n), seed=2, lo=-0.2, hi=0.2)
        C = ng.empty((m, n))
        a = A.T if op[0] == "t" else A
        b = B.T if op[1] == "t" else B
        fn = lambda: ng.dot(a, b, C, relu=True)
        work, unit = 2.0 * m * n * k, "TFLOP/s"
        algo_bytes = 2 * (m * k + k * n + m * n)
    elif name.startswith("step:"):
        # "step:alexnet:128": whole steps of the benchmark stack, every kernel launched live on one stream
        from nervanagpu_b200.convnet import ConvStack, NETWORKS
        _, net, n = name.split(":")
        ng.stream = ng.new_stream()
        stack = ConvStack(ng, NETWORKS[net], N=int(n), seed=1003)
        stack.overlap_update = False
        fn = stack.step
        work, unit = stack.flops, "TFLOP/s"
        algo_bytes = 0
    elif name.startswith("bn_"):
        rows = int(name.split("_")[1])
        A = _fill(ng, (rows, 128), seed=5, lo=0.0)
        fn = lambda: A._assign((A - ng.mean(A, axis=1)) / ng.sqrt(ng.var(A, axis=1) + 1e-3))
        algo_bytes = 2 * 2 * rows * 128
        work, unit = algo_bytes, "GB/s"
    elif name.startswith("ew_"):
        n = int(name.split("_")[1])
        A, B, C = _fill(ng, (n,), seed=1), _fill(ng, (n,), seed=2), ng.empty((n,))
        fn = lambda: C._assign(A * B + 1.5)
        algo_bytes = 3 * 2 * n
        work, unit = algo_bytes, "GB/s"
    else:
        raise SystemExit("unknown case %s" % name)
    ms = _timed(ng, fn, warm, reps)
    rate = work / (ms * 1e-3) / (1e12 if unit == "TFLOP/s" else 1e9)
    out = {"case": name, "ms": ms, "rate": rate, "unit": unit, "algorithmic_bytes": algo_bytes,
           "gbs_algorithmic": algo_bytes / (ms * 1e-3) / 1e9, "reps": reps, "warm": warm}
    print(json.dumps(out))
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("cases", nargs="+")
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--warm", type=int, default=3)
    args = ap.parse_args()
    names = []
    for c in args.cases:
        if c == "all_conv":
            names += ["%s_%s" % (l, op) for l in CONV for op in ("fprop", "bprop", "update")]
        elif c == "all_gemm":
            names += list(GEMM)
        elif c == "all_pool":
            names += ["%s_%s" % (l, op) for l in POOL for op in ("fprop", "bprop")]
        else:
            names.append(c)
    for n in names:
        run_case(n, args.warm, args.reps)


if __name__ == "__main__":
    sys.exit(main())
