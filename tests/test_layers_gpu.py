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


def test_layer_chain_forward_backward_and_sgd_match_numpy():
    """DataLayer -> ConvLayer -> PoolLayer -> FullLayer through Layer.create, one forward pass, one
    backward pass with the SGD step (nervanagpu/layers.py:87-96, 259-274, 483-502), against a numpy
    restatement. Each stage is checked on the inputs the device itself produced for it, so the
    tolerances stay those of a single kernel."""
    from oracle import reference_math as rm
    from tests._util import assert_close, rn16_tol
    ng = NervanaGPU(stochastic_round=False)
    confs = [cb._data(64, 3, 8), cb._conv(16, 3, pad=1), cb._pool(2, 2), cb._full(40)]
    data, conv, pool, full = layers = cb.build_network(ng, confs, seed=5)
    lr = -0.05
    for l in layers:
        l.learning_rate = lr
    f32 = np.float32
    I = data.fprop_out.get()
    Wc, Wf = conv.weights.get(), full.weights.get()

    x = None
    for l in layers:
        x = l.fprop(x)
    cd = rm.ConvDims(64, 3, 16, 1, 8, 8, 1, 3, 3, 0, 1, 1, 1, 1, 1)
    O1 = conv.fprop_out.get()
    ref = rm.conv_fprop_fast(cd, I, Wc, relu=True)
    assert_close(O1, ref, rn16_tol(ref, rm.conv_fprop_fast(cd, np.abs(I.astype(f32)), np.abs(Wc.astype(f32))), 27), "conv fprop")
    pd = rm.PoolDims(64, 16, 1, 8, 8, 1, 1, 2, 2, 0, 0, 0, 0, 1, 1, 2, 2)
    O2 = pool.fprop_out.get()
    assert np.array_equal(O2, rm.pool_max(pd, O1)[0].astype(np.float16))
    X2 = O2.reshape(full.nIn, 64)
    O3 = full.fprop_out.get()
    ref = rm.gemm(Wf, X2, relu=True)
    assert_close(O3, ref, rn16_tol(ref, rm.gemm_abs(Wf, X2), full.nIn), "full fprop")
    assert (O1 > 0).any() and (O3 > 0).any()

    # backward: deltas enter at the top; every layer masks them with its own ReLU output first
    rng = np.random.default_rng(9)
    E = (rng.uniform(-1, 1, full.dimO) * 0.25).astype(np.float16)
    dE = ng.array(E)
    d_full = full.bprop(dE)
    Em = (E.astype(f32) * (O3 > 0)).astype(np.float16)
    assert np.array_equal(dE.get(), Em)                                   # masked in place
    ref = rm.gemm(Wf, Em, a_t=True)                                       # weights.T @ deltas
    D3 = d_full.get()
    assert_close(D3, ref, rn16_tol(ref, rm.gemm_abs(Wf, Em, a_t=True), 40), "full bprop")
    dWf = rm.gemm(Em, X2, b_t=True).astype(np.float16).astype(f32)        # FullLayer keeps dW in fp16
    want = (Wf.astype(f32) + dWf * f32(lr)).astype(np.float16)
    got = full.weights.get()
    assert_close(got, want.astype(f32), 2.0 ** -9 * np.abs(want.astype(f32)) + abs(lr) * 2.0 ** -9 * np.abs(dWf) + 1e-6,
                 "full sgd")
    assert (got != Wf).any()

    d_pool = pool.bprop(d_full)
    D2 = d_pool.get()
    assert np.array_equal(D2, rm.pool_max(pd, O1, D3.reshape(pool.dimO))[1].astype(np.float16))

    assert conv.bprop_out is None                 # first layer above the data: no input gradient
    conv.bprop(d_pool)
    D2m = (D2.astype(f32) * (O1 > 0)).astype(np.float16)
    dWc = rm.conv_update_fast(cd, I, D2m)
    want = (Wc.astype(f32) + dWc * f32(lr)).astype(np.float16).astype(f32)
    absu = rm.conv_update_fast(cd, np.abs(I.astype(f32)), np.abs(D2m.astype(f32)))
    assert_close(conv.weights.get(), want, 2.0 ** -9 * np.abs(want) + abs(lr) * 64 * 64 * 2.0 ** -23 * absu + 1e-6,
                 "conv sgd")
    assert (conv.weights.get() != Wc).any()


def test_deconv_layer_is_the_transposed_convolution():
    """DeconvLayer (nervanagpu/layers.py:509-537) takes the output size of the equivalent
    convolution; its forward pass is that convolution's backward pass and vice versa."""
    from oracle import reference_math as rm
    from tests._util import assert_close, f32_tol, rn16_tol
    ng = NervanaGPU(stochastic_round=False)
    N, C, K, P, Q, R, S, pad, stride = 64, 16, 32, 6, 6, 4, 4, 1, 2
    layer = ng.deconv_layer(np.float16, N, C, K, P, Q, R, S, pad_h=pad, pad_w=pad, str_h=stride, str_w=stride)
    H = (P - 1) * stride - 2 * pad + R
    assert layer.DHW == (1, H, H) and layer.MPQ == (1, P, Q) and layer.dimO == (K, 1, P, Q, N)
    assert layer.nOut == C * H * H and str(layer).startswith("DeconvLayer")
    cd = rm.ConvDims(N, C, K, 1, H, H, 1, R, S, 0, pad, pad, 1, stride, stride)
    rng = np.random.default_rng(21)
    W = rng.normal(0, 0.1, layer.dimF).astype(np.float16)
    X = rng.uniform(-1, 1, layer.dimO).astype(np.float16)          # the deconvolution's input has K maps
    G = rng.uniform(-1, 1, layer.dimI).astype(np.float16)          # deltas arrive with C maps
    f32 = np.float32
    layer.weights = ng.array(W)
    layer.updat_out = ng.empty(layer.dimF, dtype=np.float32)
    layer.init_activations()
    layer.bprop_out = ng.empty(layer.dimO)
    layer.learning_rate = 0.0
    out = layer.fprop(ng.array(X)).get()
    ref = rm.conv_bprop_fast(cd, W, X)
    assert out.shape == layer.dimI
    assert_close(out, ref, rn16_tol(ref, rm.conv_bprop_fast(cd, np.abs(W.astype(f32)), np.abs(X.astype(f32))),
                                    K * R * S), "deconv fprop")
    back = layer.bprop(ng.array(G)).get()
    ref = rm.conv_fprop_fast(cd, G, W)
    assert_close(back, ref, rn16_tol(ref, rm.conv_fprop_fast(cd, np.abs(G.astype(f32)), np.abs(W.astype(f32))),
                                     C * R * S), "deconv bprop")
    ref = rm.conv_update_fast(cd, G, X)
    assert_close(layer.updat_out.get(), ref,
                 f32_tol(rm.conv_update_fast(cd, np.abs(G.astype(f32)), np.abs(X.astype(f32))), P * Q * N), "deconv update")
