"""Whole-network forward / backward timing through the Layer classes.

    python -m nervanagpu_b200.convnet_benchmarks [--nets Alexnet,VGG] [--loops 10] [--layer-bench] [--stats]

The counterpart of the reference's benchmarks/convnet-benchmarks.py:250-403: each network is a list
of layer configurations turned into Layer objects by Layer.create, delta buffers are shared between
alternating layers, the initial weights are scaled so that activations stay near 1, and `loops`
iterations of fprop over all layers and bprop (deltas, weight update and SGD step, in reverse) are
timed with events. Output lines have the reference's form ("Avg(10) fprop: ... msecs ... gflops"),
flops per layer from Layer.flops with the backward pass counted twice.

Networks: the convolution/pooling/fully-connected stacks of AlexNet (one-column variant), Overfeat
(fast), VGG model A and VGG model E as the public convnet-benchmarks lists them, and GoogLeNet (v1,
nine Inception modules), fp16 only (fp32 layers are outside this library). The per-layer grid hints of the reference's tables tuned its
Maxwell kernels and have no meaning here.
"""
import argparse
import ctypes

import numpy as np

from . import NervanaGPU, _lib
from .layers import ConvLayer, DataLayer, FullLayer, Inception, Layer, PoolLayer


def _conv(K, R, pad=0, stride=1):
    return {"layer": ConvLayer, "K": K, "R": R, "S": R, "pad_h": pad, "pad_w": pad, "str_h": stride, "str_w": stride}


def _pool(R, stride):
    return {"layer": PoolLayer, "op": "max", "R": R, "S": R, "str_h": stride, "str_w": stride}


def _full(n_out):
    return {"layer": FullLayer, "nOut": n_out}


def _data(N, C, H):
    return {"layer": DataLayer, "N": N, "C": C, "H": H, "W": H}


def _inception(n1x1, red3, n3x3, red5, n5x5, proj):
    """GoogLeNet module: 1x1 | 1x1 -> 3x3 | 1x1 -> 5x5 | 3x3 max-pool (stride 1) -> 1x1."""
    pool = dict(_pool(3, 1), pad_h=1, pad_w=1)
    return {"layer": Inception, "partitions": [
        [_conv(n1x1, 1)],
        [_conv(red3, 1), _conv(n3x3, 3, pad=1)],
        [_conv(red5, 1), _conv(n5x5, 5, pad=2)],
        [pool, _conv(proj, 1)],
    ]}


def _pool_same(R, stride):
    # padded so that 112 -> 56 -> 28 -> 14 -> 7, the map sizes the published network uses
    return dict(_pool(R, stride), pad_h=1, pad_w=1)


_CLASSIFIER = [_full(3072), _full(3072), _full(1000)]


def _vgg(blocks):
    layers = [_data(64, 3, 224)]
    for convs, K in blocks:
        layers += [_conv(K, 3, pad=1) for _ in range(convs)]
        layers.append(_pool(2, 2))
    return layers + _CLASSIFIER


NETWORKS = {
    # name: (untimed warm-up iterations, layer configurations)
    "Alexnet": (5, [_data(128, 3, 224), _conv(64, 11, pad=2, stride=4), _pool(3, 2), _conv(192, 5, pad=2), _pool(3, 2),
                    _conv(384, 3, pad=1), _conv(256, 3, pad=1), _conv(256, 3, pad=1), _pool(3, 2)] + _CLASSIFIER),
    "Overfeat": (1, [_data(128, 3, 231), _conv(96, 11, stride=4), _pool(2, 2), _conv(256, 5), _pool(2, 2),
                     _conv(512, 3, pad=1), _conv(1024, 3, pad=1), _conv(1024, 3, pad=1), _pool(2, 2)] + _CLASSIFIER),
    "GoogLeNet1": (1, [_data(128, 3, 224), _conv(64, 7, pad=3, stride=2), _pool_same(3, 2), _conv(64, 1),
                       _conv(192, 3, pad=1), _pool_same(3, 2),
                       _inception(64, 96, 128, 16, 32, 32), _inception(128, 128, 192, 32, 96, 64), _pool_same(3, 2),
                       _inception(192, 96, 208, 16, 48, 64), _inception(160, 112, 224, 24, 64, 64),
                       _inception(128, 128, 256, 24, 64, 64), _inception(112, 144, 288, 32, 64, 64),
                       _inception(256, 160, 320, 32, 128, 128), _pool_same(3, 2),
                       _inception(256, 160, 320, 32, 128, 128), _inception(384, 192, 384, 48, 128, 128),
                       _pool(7, 1), _full(1000)]),
    "VGG": (1, _vgg([(1, 64), (1, 128), (2, 256), (2, 512), (2, 512)])),
    "VGG_E": (1, _vgg([(2, 64), (2, 128), (4, 256), (4, 512), (4, 512)])),
}


class _Stopwatch(object):
    def __init__(self, ng):
        self.ng = ng
        self.a, self.b = ctypes.c_void_p(), ctypes.c_void_p()
        _lib.check(ng.lib.ng_event_create(ctypes.byref(self.a)))
        _lib.check(ng.lib.ng_event_create(ctypes.byref(self.b)))

    def start(self):
        _lib.check(self.ng.lib.ng_event_record(self.a, self.ng.stream))

    def stop_ms(self):
        lib = self.ng.lib
        _lib.check(lib.ng_event_record(self.b, self.ng.stream))
        _lib.check(lib.ng_event_sync(self.b))
        ms = ctypes.c_float()
        _lib.check(lib.ng_event_elapsed_ms(self.a, self.b, ctypes.byref(ms)))
        return ms.value


def build_network(ng, confs, dtype=np.float16, zeros=False, seed=0):
    """Layer objects with activations, weights and (shared) delta buffers in place."""
    layers, prev = [], None
    for conf in confs:
        prev = Layer.create(ng, conf, prev, dtype)
        layers.append(prev)
    # the two largest delta buffers and the largest weight-gradient buffer are shared by all layers
    deltas = max((l for i, l in enumerate(layers) if i > 1), key=lambda l: l.sizeI)
    widest = max(layers, key=lambda l: l.sizeF)
    shared_deltas = [ng.empty(deltas.dimI, dtype=deltas.dtype), ng.empty(deltas.dimI, dtype=deltas.dtype)]
    shared_updates = ng.empty(widest.dimF, dtype=np.float32)
    rng = np.random.RandomState(seed)
    for i, layer in enumerate(layers):
        layer.init_activations()
        layer.init_weights(shared=shared_updates, zeros=zeros, rng=rng)
        if i > 1:
            layer.init_deltas(shared=shared_deltas)
    if zeros:
        layers[0].init_data()
    else:
        layers[0].init_data(rng.uniform(0.0, 1.0, layers[0].dimO))
        bench, ng.bench = ng.bench, False
        x = None
        for layer in layers:          # one pass that scales each layer's weights from its activation mean
            x = layer.fprop(x, scale_weights=.5)
        ng.bench = bench
    return layers


def run_network(ng, name, loops=10, stats=False, zeros=False, out=print):
    warmup, confs = NETWORKS[name]
    title = "%s (dtype=float16, N=%d)" % (name, confs[0]["N"])
    out("------------------------------------------------")
    out("Benchmarking: " + title)
    out("------------------------------------------------")
    layers = build_network(ng, confs, zeros=zeros)
    watch = _Stopwatch(ng)
    totals = {"fprop": [0.0, 0.0], "bprop": [0.0, 0.0]}
    for it in range(loops + warmup):
        shown = max(it - warmup + 1, 0)
        watch.start()
        flops, x = 0, None
        for layer in layers:
            x = layer.fprop(x)
            flops += layer.flops
            if stats:
                layer.fprop_stats()
        ms = watch.stop_ms()
        out("fprop(%2d): %8.3f msecs %8.3f gflops" % (shown, ms, flops / (ms * 1e6)))
        if shown > 0:
            totals["fprop"][0] += ms
            totals["fprop"][1] += flops
        watch.start()
        flops = 0
        for layer in layers[:0:-1]:
            x = layer.bprop(x)
            flops += layer.flops * 2
            if stats:
                layer.bprop_stats()
        ms = watch.stop_ms()
        out("bprop(%2d): %8.3f msecs %8.3f gflops" % (shown, ms, flops / (ms * 1e6)))
        if shown > 0:
            totals["bprop"][0] += ms
            totals["bprop"][1] += flops
    result = {}
    if loops > 0:
        out("---------------------------------------------")
        out(title + " Results:")
        out("---------------------------------------------")
        f_ms, f_fl = totals["fprop"]
        b_ms, b_fl = totals["bprop"]
        for label, ms, fl in (("fprop", f_ms, f_fl), ("bprop", b_ms, b_fl), ("total", f_ms + b_ms, f_fl + b_fl)):
            out("Avg(%d) %s: %8.3f msecs %.3f gflops" % (loops, label, ms / loops, fl / (ms * 1e6)))
            result[label] = (ms / loops, fl / (ms * 1e6))
        out("")
    return result


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--nets", default="Alexnet,Overfeat,VGG,GoogLeNet1,VGG_E")
    ap.add_argument("--loops", type=int, default=10)
    ap.add_argument("--layer-bench", action="store_true", help="print the time of every conv / pool / GEMM call")
    ap.add_argument("--stats", action="store_true", help="print activation / delta / update statistics per layer")
    ap.add_argument("--zeros", action="store_true", help="all-zero data and weights")
    args = ap.parse_args()
    ng = NervanaGPU(stochastic_round=False, bench=args.layer_bench)
    for name in args.nets.split(","):
        if name not in NETWORKS:
            raise SystemExit("unknown network %s (have: %s)" % (name, ", ".join(sorted(NETWORKS))))
        run_network(ng, name, loops=args.loops, stats=args.stats, zeros=args.zeros)


if __name__ == "__main__":
    main()
