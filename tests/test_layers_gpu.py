"""Layer containers on the device: the Inception module's concatenation and delta sum (B200 only)."""
import numpy as np
import pytest

from nervanagpu_b200 import NervanaGPU
from nervanagpu_b200 import convnet_benchmarks as cb
from nervanagpu_b200.layers import Inception

pytestmark = pytest.mark.gpu


def _tiny_network(ng):
    pool = dict(cb._pool(3, 1), pad_h=1, pad_w=1)
    module = {"layer": Inception, "partitions": [
        [cb._conv(8, 1)],
        [cb._conv(8, 1), cb._conv(16, 3, pad=1)],
        [pool, cb._conv(8, 1)],
    ]}
    confs = [cb._data(64, 3, 8), cb._conv(16, 3, pad=1), module, cb._full(40)]
    return cb.build_network(ng, confs, seed=3)


def test_inception_concatenates_branches_and_sums_their_deltas():
    ng = NervanaGPU(stochastic_round=False)
    layers = _tiny_network(ng)
    module = layers[2]
    assert isinstance(module, Inception) and module.K == 32 and module.dimO == (32, 1, 8, 8, 64)
    x = None
    for layer in layers:
        x = layer.fprop(x)
    out = module.fprop_out.get()
    k0 = 0
    for part in module.partitions:
        last = part[-1]
        assert np.array_equal(out[k0:k0 + last.K], last.fprop_out.get())      # views of one buffer
        k0 += last.K
    assert np.abs(out.astype(np.float32)).sum() > 0
    x = layers[3].bprop(x)
    got = module.bprop(x).get()      # read before the layer below masks it in place
    # each branch again on its own (learning rate 0: nothing changes between the runs), then the
    # same fp16 running sum the container forms
    deltas_in = layers[3].bprop_out.reshape(module.dimO)
    parts, k0 = [], 0
    for part in module.partitions:
        scratch = ng.empty(module.dimI)
        saved, part[0].bprop_out = part[0].bprop_out, scratch
        d = deltas_in[k0:k0 + part[-1].K]
        k0 += part[-1].K
        for layer in part[::-1]:
            d = layer.bprop(d)
        part[0].bprop_out = saved
        parts.append(scratch.get().astype(np.float32))
    want = parts[0].astype(np.float16)
    for d in parts[1:]:
        want = (want.astype(np.float32) + d).astype(np.float16)
    assert np.array_equal(got, want)
    assert all(np.abs(d).sum() > 0 for d in parts)


def test_googlenet_runs_through_the_driver():
    lines = []
    res = cb.run_network(NervanaGPU(stochastic_round=False), "GoogLeNet1", loops=1, out=lines.append)
    assert res["total"][0] > 0 and np.isfinite(res["total"][1])
