"""The three convolution passes and max-pooling at the sizes of the benchmark configurations
(AlexNet N=128, VGG model A N=64, the 3-D layer N=32) against the numpy oracle (B200 only).

Whole tensors are compared where the oracle's patch matrix fits in host memory and a pass costs a
few tens of GFLOP (every AlexNet layer); the larger layers are compared at a fixed random sample
of output pixels (forward), input positions (backward) and filter taps (update), each through the
per-position arithmetic of the reference's validation loop (benchmarks/conv_test.py:147-167).
Pooling is bit-exact against benchmarks/pool_test.py:117-140.

Tolerances (also in tests/_util.py):
  forward / backward   fp16 round-to-nearest result of a dot product of length k:
                       |d| <= 2^-10 |ref| + k 2^-24 sum|a||b| + 2^-24
                       (whole tensors bound sum|a||b| by the product of the operands' 2-norms)
  update               fp32 result of a reduction over up to 3.2 million terms, summed in another
                       order than the oracle's BLAS call. The worst-case bound k 2^-23 sum|a||b| says
                       nothing at that length, so the test uses the random-walk estimate of both
                       sides' rounding noise instead: |d| <= 16 * 2^-24 * ||a||_2 ||b||_2.
                       A dropped tap, chunk or partition is off by percents of ||a|| ||b|| / sqrt(k).
"""
import numpy as np
import pytest

from nervanagpu_b200 import _lib
from oracle import reference_math as rm
from tests._util import assert_close, rn16_tol

pytestmark = pytest.mark.gpu

# (N, C, K, D, H, W, T, R, S, pad_d, pad_h, pad_w, str_d, str_h, str_w)
ALEXNET = {
    "conv1": (128, 3, 64, 1, 224, 224, 1, 11, 11, 0, 2, 2, 1, 4, 4),
    "conv2": (128, 64, 192, 1, 27, 27, 1, 5, 5, 0, 2, 2, 1, 1, 1),
    "conv3": (128, 192, 384, 1, 13, 13, 1, 3, 3, 0, 1, 1, 1, 1, 1),
    "conv4": (128, 384, 256, 1, 13, 13, 1, 3, 3, 0, 1, 1, 1, 1, 1),
    "conv5": (128, 256, 256, 1, 13, 13, 1, 3, 3, 0, 1, 1, 1, 1, 1),
}


def _vgg(C, K, HW, N=64):
    return (N, C, K, 1, HW, HW, 1, 3, 3, 0, 1, 1, 1, 1, 1)


SAMPLED = {
    # name: (configuration, output pixels, input positions, filter taps)
    "vgg_3_64_224": (_vgg(3, 64, 224), 4096, 4096, 9),
    "vgg_64_128_112": (_vgg(64, 128, 112), 4096, 4096, 3),
    "vgg_128_256_56": (_vgg(128, 256, 56), 512, 512, 2),
    "vgg_256_256_56": (_vgg(256, 256, 56), 384, 384, 2),
    "vgg_256_512_28": (_vgg(256, 512, 28), 256, 256, 2),
    "vgg_512_512_28": (_vgg(512, 512, 28), 192, 192, 2),
    "vgg_512_512_14": (_vgg(512, 512, 14), 196, 196, 2),
    "config5_3d_64_64": ((32, 64, 64, 16, 56, 56, 3, 3, 3, 1, 1, 1, 1, 1, 1), 4096, 4096, 3),
}


def _inputs(cd, seed):
    rng = np.random.default_rng(seed)
    I = rng.uniform(0, 1, cd.dimI).astype(np.float16)
    F = rng.normal(0, 0.01, cd.dimF).astype(np.float16)
    E = (rng.uniform(-1, 1, cd.dimO) * 0.125).astype(np.float16)
    return I, F, E


def _run(ng, cfg, I, F, E):
    layer = ng.conv_layer(np.float16, *cfg)
    dI, dF, dE = ng.array(I), ng.array(F), ng.array(E)
    dO = ng.empty(layer.dimO)
    ng.fprop_conv(layer, dI, dF, dO, relu=True)
    O = dO.get()
    del dO
    dB = ng.empty(layer.dimI)
    ng.bprop_conv(layer, dF, dE, dB)
    B = dB.get()
    del dB
    dU = ng.empty(layer.dimF, dtype=np.float32)
    ng.update_conv(layer, dI, dE, dU)
    U = dU.get()
    _lib.check(ng.lib.ng_sync())
    return O, B, U


def _norm_bounds(cd, I, F, E):
    """Upper bounds of sum|a||b| for every output of the forward and backward pass (Cauchy-Schwarz:
    norm of the filter slice times norm of the patch), and the norms of the update's operands."""
    T, R, S = cd.TRS
    I32, F32, E32 = I.astype(np.float32), F.astype(np.float32), E.astype(np.float32)
    one = rm.ConvDims(cd.N, 1, 1, *cd.DHW, T, R, S, *cd.padding, *cd.strides)
    ones = np.ones(one.dimF, np.float32)
    patch = np.sqrt(rm.conv_fprop_fast(one, (I32 ** 2).sum(axis=0, keepdims=True), ones))      # (1,M,P,Q,N)
    f_k = np.sqrt((F32 ** 2).sum(axis=(0, 1, 2, 3)))                                           # (K,)
    fprop = f_k[:, None, None, None, None] * patch
    reach = np.sqrt(rm.conv_bprop_fast(one, ones, (E32 ** 2).sum(axis=0, keepdims=True)))      # (1,D,H,W,N)
    f_c = np.sqrt((F32 ** 2).sum(axis=(1, 2, 3, 4)))                                           # (C,)
    bprop = f_c[:, None, None, None, None] * reach
    i_c = np.sqrt((I32.astype(np.float64) ** 2).sum(axis=(1, 2, 3, 4)))                        # (C,)
    e_k = np.sqrt((E32.astype(np.float64) ** 2).sum(axis=(1, 2, 3, 4)))                        # (K,)
    return fprop, bprop, i_c, e_k


def _rms_rel(got, ref):
    got = np.asarray(got, dtype=np.float32)
    return float(np.sqrt(np.mean((got - ref) ** 2, dtype=np.float64) / np.mean(ref ** 2, dtype=np.float64)))


# Besides the element-wise bounds, the error as a whole must look like rounding noise: one fp16
# rounding is at most 2^-11 relative (rms about 2^-12 of the values). The fp32 weight gradients
# differ from a double-precision sum by the accumulators' own rounding: the tensor cores add each
# K=16 step into the fp32 accumulator with truncation, so a chain of several hundred steps ends
# up to 2e-4 below the exact magnitude (measured on the 3-D layer, 1.6 million terms per output,
# 6.4e-5 rms; the reference's own fp32 FFMA chains have a rounding error of the same order).
RMS_FP16, RMS_FP32 = 2.0 ** -11, 2.0 ** -12


def _update_tol(i_c, e_k):
    return (16.0 * 2.0 ** -24 * i_c[:, None] * e_k[None, :]).astype(np.float32) + 1e-30


@pytest.mark.parametrize("name", sorted(ALEXNET))
def test_alexnet_layers_whole_tensors(ng, name):
    cfg = ALEXNET[name]
    cd = rm.ConvDims(*cfg)
    T, R, S = cd.TRS
    I, F, E = _inputs(cd, 1003)
    O, B, U = _run(ng, cfg, I, F, E)
    fb, bb, i_c, e_k = _norm_bounds(cd, I, F, E)
    ref = rm.conv_fprop_fast(cd, I, F, relu=True)
    assert_close(O, ref, rn16_tol(ref, fb, cd.C * T * R * S), name + " fprop")
    assert _rms_rel(O, ref) <= RMS_FP16
    del ref, fb
    ref = rm.conv_bprop_fast(cd, F, E)
    assert_close(B, ref, rn16_tol(ref, bb, cd.K * T * R * S), name + " bprop")
    assert _rms_rel(B, ref) <= RMS_FP16
    del ref, bb
    ref = rm.conv_update_fast(cd, I, E)
    assert_close(U, ref, _update_tol(i_c, e_k)[:, None, None, None, :], name + " update")
    assert _rms_rel(U, ref) <= RMS_FP32
    assert np.abs(ref).mean() > 64 * _update_tol(i_c, e_k).mean()      # the tolerance is far below the values


def _sample(rng, dims, count):
    total = int(np.prod(dims))
    flat = rng.choice(total, size=min(count, total), replace=False)
    corners = [0, total - 1, dims[2] - 1, total - dims[2]]
    flat = np.unique(np.concatenate([flat, corners]))
    return [tuple(int(v) for v in np.unravel_index(i, dims)) for i in flat]


@pytest.mark.parametrize("name", sorted(SAMPLED))
def test_large_layers_at_sampled_positions(ng, name):
    cfg, n_pix, n_pos, n_taps = SAMPLED[name]
    cd = rm.ConvDims(*cfg)
    T, R, S = cd.TRS
    I, F, E = _inputs(cd, 1004)
    O, B, U = _run(ng, cfg, I, F, E)
    rng = np.random.default_rng(7)

    pix = _sample(rng, cd.MPQ, n_pix)
    ref = rm.conv_fprop_pixels(cd, I, F, pix, relu=True)
    absd = rm.conv_fprop_pixels(cd, I, F, pix, absolute=True)
    got = np.stack([O[:, m, p, q, :] for m, p, q in pix])
    assert_close(got, ref, rn16_tol(ref, absd, cd.C * T * R * S), name + " fprop")
    assert _rms_rel(got, ref) <= RMS_FP16

    pos = _sample(rng, cd.DHW, n_pos)
    ref = rm.conv_bprop_pixels(cd, F, E, pos)
    absd = rm.conv_bprop_pixels(cd, F, E, pos, absolute=True)
    got = np.stack([B[:, z, y, x, :] for z, y, x in pos])
    assert_close(got, ref, rn16_tol(ref, absd, cd.K * T * R * S), name + " bprop")
    assert _rms_rel(got, ref) <= RMS_FP16

    all_taps = [(t, r, s) for t in range(T) for r in range(R) for s in range(S)]
    picks = sorted(set([0, len(all_taps) - 1] + [int(i) for i in rng.choice(len(all_taps), n_taps, replace=False)]))
    taps = [all_taps[i] for i in picks[:max(n_taps, 2)]]
    ref = rm.conv_update_taps(cd, I, E, taps, dtype=np.float64)   # millions of terms: sum in double
    i_c = np.sqrt((I.astype(np.float64) ** 2).sum(axis=(1, 2, 3, 4)))
    e_k = np.sqrt((E.astype(np.float64) ** 2).sum(axis=(1, 2, 3, 4)))
    got = np.stack([U[:, t, r, s, :] for t, r, s in taps])
    assert_close(got, ref, _update_tol(i_c, e_k)[None], name + " update")
    assert _rms_rel(got, ref) <= RMS_FP32
    assert np.abs(ref).mean() > 64 * _update_tol(i_c, e_k).mean()


POOLS = {
    # (N, C, D, H, W, J, T, R, S, pad_j, pad_d, pad_h, pad_w, str_j, str_d, str_h, str_w)
    "alexnet_pool1": (128, 64, 1, 55, 55, 1, 1, 3, 3, 0, 0, 0, 0, 1, 1, 2, 2),
    "alexnet_pool2": (128, 192, 1, 27, 27, 1, 1, 3, 3, 0, 0, 0, 0, 1, 1, 2, 2),
    "alexnet_pool5": (128, 256, 1, 13, 13, 1, 1, 3, 3, 0, 0, 0, 0, 1, 1, 2, 2),
    "vgg_pool1": (64, 64, 1, 224, 224, 1, 1, 2, 2, 0, 0, 0, 0, 1, 1, 2, 2),
    "vgg_pool2": (64, 128, 1, 112, 112, 1, 1, 2, 2, 0, 0, 0, 0, 1, 1, 2, 2),
    "vgg_pool3": (64, 256, 1, 56, 56, 1, 1, 2, 2, 0, 0, 0, 0, 1, 1, 2, 2),
    "vgg_pool4": (64, 512, 1, 28, 28, 1, 1, 2, 2, 0, 0, 0, 0, 1, 1, 2, 2),
    "vgg_pool5": (64, 512, 1, 14, 14, 1, 1, 2, 2, 0, 0, 0, 0, 1, 1, 2, 2),
    "config5_pool_jtrs_2222": (32, 64, 16, 56, 56, 2, 2, 2, 2, 0, 0, 0, 0, 2, 2, 2, 2),
}


@pytest.mark.parametrize("name", sorted(POOLS))
def test_pools_bit_exact_at_full_size(ng, name):
    cfg = POOLS[name]
    pd = rm.PoolDims(*cfg)
    rng = np.random.default_rng(1005)
    # a ReLU-like input with many equal values (ties decide the argmax) and an error tensor
    I = (np.maximum(rng.integers(-6, 26, pd.dimI, dtype=np.int8), 0) / 16.0).astype(np.float16)
    E = rng.uniform(-1, 1, pd.dimO).astype(np.float16)
    layer = ng.pool_layer(np.float16, "max", *cfg)
    dI, dE = ng.array(I), ng.array(E)
    dO, dB = ng.empty(layer.dimO), ng.empty(layer.dimI)
    ng.fprop_pool(layer, dI, dO)
    ng.bprop_pool(layer, dI, dE, dB)
    O, B = dO.get(), dB.get()
    refO, refB = rm.pool_max_fast(pd, I, E)
    assert np.array_equal(O, refO.astype(np.float16)), name + " fprop"
    assert np.array_equal(B, refB.astype(np.float16)), name + " bprop"
