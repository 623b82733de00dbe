"""fprop_conv / bprop_conv / update_conv against the reference's numpy path (B200 only)."""
import numpy as np
import pytest

from nervanagpu_b200 import _lib
from oracle import reference_math as rm
from tests._util import assert_close, f32_tol, golden, golden_names, rn16_tol

pytestmark = pytest.mark.gpu

PATHS = {"auto": _lib.NG_PATH_AUTO, "tensor": _lib.NG_PATH_TENSOR, "simt": _lib.NG_PATH_SIMT,
         "im2col": _lib.NG_PATH_IM2COL}


def _layer(ng, cfg, path="auto"):
    layer = ng.conv_layer(np.float16, *cfg)
    layer.path = PATHS[path]
    return layer


def _abs_terms(cd, I, F, E):
    """sum |a||b| of each output's dot product, for the accumulation-error bound."""
    aI, aF, aE = np.abs(I.astype(np.float32)), np.abs(F.astype(np.float32)), np.abs(E.astype(np.float32))
    return rm.conv_fprop_fast(cd, aI, aF), rm.conv_bprop_fast(cd, aF, aE), rm.conv_update_fast(cd, aI, aE)


def _run_all(ng, layer, I, F, E, relu=False, alpha=1.0, ops="fbu"):
    dI, dF, dE = ng.array(I), ng.array(F), ng.array(E)
    out = {}
    if "f" in ops:
        dO = ng.empty(layer.dimO)
        ng.fprop_conv(layer, dI, dF, dO, alpha=alpha, relu=relu)
        out["O"] = dO.get()
    if "b" in ops:
        dB = ng.empty(layer.dimI)
        ng.bprop_conv(layer, dF, dE, dB, alpha=alpha)
        out["gradI"] = dB.get()
    if "u" in ops:
        dU = ng.empty(layer.dimF, dtype=np.float32)
        ng.update_conv(layer, dI, dE, dU, alpha=alpha)
        out["gradF"] = dU.get()
    return out


def _check(cd, got, I, F, E, ref, what):
    T, R, S = cd.TRS
    aO, aB, aU = _abs_terms(cd, I, F, E)
    M, P, Q = cd.MPQ
    if "O" in got:
        assert_close(got["O"], ref["O"], rn16_tol(ref["O"], aO, cd.C * T * R * S), what + " fprop")
    if "gradI" in got:
        assert_close(got["gradI"], ref["gradI"], rn16_tol(ref["gradI"], aB, cd.K * T * R * S), what + " bprop")
    if "gradF" in got:
        assert_close(got["gradF"], ref["gradF"], f32_tol(aU, M * P * Q * cd.N), what + " update")


@pytest.mark.parametrize("name", golden_names("conv_"))
@pytest.mark.parametrize("path", ["auto", "simt"])
def test_golden_vectors_of_the_reference_numpy_path(ng, name, path):
    g = golden(name)
    cfg = [int(v) for v in g["cfg"]]
    cd = rm.ConvDims(*cfg)
    got = _run_all(ng, _layer(ng, cfg, path), g["I"], g["F"], g["E"])
    _check(cd, got, g["I"], g["F"], g["E"], g, "%s/%s" % (name, path))


CASES = {
    # name: (N, C, K, D, H, W, T, R, S, pad_d, pad_h, pad_w, str_d, str_h, str_w)
    "c64_3x3_n64": (64, 64, 128, 1, 8, 8, 1, 3, 3, 0, 1, 1, 1, 1, 1),
    "c3_3x3_n64_first_layer": (64, 3, 64, 1, 12, 12, 1, 3, 3, 0, 1, 1, 1, 1, 1),
    "c16_5x5_stride2_n128": (128, 16, 32, 1, 13, 13, 1, 5, 5, 0, 2, 2, 1, 2, 2),
    "c96_3x3_n32_flattened": (32, 96, 64, 1, 8, 8, 1, 3, 3, 0, 1, 1, 1, 1, 1),
    "c64_3d_n32": (32, 64, 64, 4, 6, 6, 3, 3, 3, 1, 1, 1, 1, 1, 1),
    "c3_11x11_stride4_n64_alexnet1": (64, 3, 64, 1, 35, 35, 1, 11, 11, 0, 2, 2, 1, 4, 4),
    "c130_k200_ragged_channels": (64, 130, 200, 1, 7, 7, 1, 3, 3, 0, 0, 0, 1, 1, 1),
    "c32_1x1": (64, 32, 48, 1, 5, 5, 1, 1, 1, 0, 0, 0, 1, 1, 1),
    "c8_n16_flattened_q8": (16, 8, 16, 1, 8, 8, 1, 3, 3, 0, 1, 1, 1, 1, 1),
    "stride_h_only": (64, 16, 16, 1, 9, 8, 1, 3, 3, 0, 1, 1, 1, 2, 1),
    # update: two 48-row taps stacked per accumulator, 192-column tiles
    "c48_k384_stacked_taps": (64, 48, 384, 1, 6, 6, 1, 3, 3, 0, 1, 1, 1, 1, 1),
    "c64_k192_5x5_n128": (128, 64, 192, 1, 7, 7, 1, 5, 5, 0, 2, 2, 1, 1, 1),
    # tap blocks with two image groups per pixel (one box per pixel), update with exchanged operands
    "c3_11x11_stride4_n128": (128, 3, 64, 1, 27, 27, 1, 11, 11, 0, 2, 2, 1, 4, 4),
    # 256 output rows: filter halves as single boxes, column tiles as single boxes (N = 64),
    # and a width (6) that makes some tiles straddle image rows
    "c64_k256_w6_merged_boxes": (64, 64, 256, 1, 6, 6, 1, 3, 3, 0, 1, 1, 1, 1, 1),
    # K = 96: the first-layer update keeps the filters on the MMA rows (K <= 128), one column tile
    "c3_7x7_stride2_k96": (64, 3, 96, 1, 21, 21, 1, 7, 7, 0, 3, 3, 1, 2, 2),
}


# Per-GPU shapes of a minibatch that is split over 2 / 4 / 8 GPUs (AlexNet 128 -> 64/32/16, VGG model A
# 64 -> 32/16/8): with fewer than 64 images a 64-element chunk is several pixels of one image row, and
# rows that are not a multiple of 64 elements (13 x 32, 27 x 16, 14 x 8, ...) are padded to whole chunks.
SHARDED = {
    "alexnet_conv2_n32": (32, 64, 192, 1, 27, 27, 1, 5, 5, 0, 2, 2, 1, 1, 1),
    "alexnet_conv2_n16": (16, 64, 192, 1, 27, 27, 1, 5, 5, 0, 2, 2, 1, 1, 1),
    "alexnet_conv3_n32": (32, 192, 384, 1, 13, 13, 1, 3, 3, 0, 1, 1, 1, 1, 1),
    "alexnet_conv3_n16": (16, 192, 384, 1, 13, 13, 1, 3, 3, 0, 1, 1, 1, 1, 1),
    "alexnet_conv4_n16": (16, 384, 256, 1, 13, 13, 1, 3, 3, 0, 1, 1, 1, 1, 1),
    "alexnet_conv5_n32": (32, 256, 256, 1, 13, 13, 1, 3, 3, 0, 1, 1, 1, 1, 1),
    "vgg_64_128_n8_w20": (8, 64, 128, 1, 20, 20, 1, 3, 3, 0, 1, 1, 1, 1, 1),
    "vgg_256_512_28_n8": (8, 256, 512, 1, 28, 28, 1, 3, 3, 0, 1, 1, 1, 1, 1),
    "vgg_512_512_14_n8": (8, 512, 512, 1, 14, 14, 1, 3, 3, 0, 1, 1, 1, 1, 1),
    "vgg_512_512_14_n16": (16, 512, 512, 1, 14, 14, 1, 3, 3, 0, 1, 1, 1, 1, 1),
    "vgg_512_512_14_n32": (32, 512, 512, 1, 14, 14, 1, 3, 3, 0, 1, 1, 1, 1, 1),
    # no padding (Q < W): the tail of a row's last chunk reads real pixels of the next columns
    "valid_conv_n24_q9": (24, 32, 64, 1, 11, 11, 1, 3, 3, 0, 0, 0, 1, 1, 1),
    # 3-D, one image row shorter than a chunk
    "c32_3d_n8_w5": (8, 32, 32, 3, 5, 5, 3, 3, 3, 1, 1, 1, 1, 1, 1),
}


def _inputs(cd, seed):
    rng = np.random.default_rng(seed)
    I = rng.uniform(0, 1, cd.dimI).astype(np.float16)
    F = rng.normal(0, 0.1, cd.dimF).astype(np.float16)
    E = (rng.uniform(-1, 1, cd.dimO) * 0.125).astype(np.float16)
    return I, F, E


@pytest.mark.parametrize("name", sorted(CASES))
def test_tensor_core_path_matches_oracle(ng, name):
    cfg = CASES[name]
    cd = rm.ConvDims(*cfg)
    I, F, E = _inputs(cd, 1003)
    ref = {"O": rm.conv_fprop_fast(cd, I, F, alpha=0.5, relu=True), "gradI": rm.conv_bprop_fast(cd, F, E, alpha=0.5),
           "gradF": rm.conv_update_fast(cd, I, E, alpha=0.5)}
    got = _run_all(ng, _layer(ng, cfg, "tensor"), I, F, E, relu=True, alpha=0.5)
    _check(cd, got, I, F, E, ref, name)
    assert (got["O"] >= 0).all()


BLOCKED = ["c64_3x3_n64", "c96_3x3_n32_flattened", "c64_3d_n32", "c130_k200_ragged_channels", "stride_h_only",
           "c48_k384_stacked_taps", "c64_k192_5x5_n128", "c64_k256_w6_merged_boxes"]


@pytest.mark.parametrize("name", BLOCKED)
def test_channel_blocked_copies_change_nothing(ng, lib, name):
    """Activation tensors whose channel planes are larger than a page are read through a copy in
    (z, y, channel, x, n) order (the "chan_block" tuning field: 2 = every shape, 0 = never). The
    product reads the same values in the same order either way: results are equal bit for bit,
    for every kind of tensor map (per pixel, flattened rows, merged boxes, strided rows)."""
    cfg = CASES[name]
    cd = rm.ConvDims(*cfg)
    I, F, E = _inputs(cd, 1005)
    try:
        assert lib.ng_tune(b"chan_block", 0) == 0
        plain = _run_all(ng, _layer(ng, cfg, "tensor"), I, F, E, relu=True, alpha=0.5)
        assert lib.ng_tune(b"chan_block", 2) == 0
        blocked = _run_all(ng, _layer(ng, cfg, "tensor"), I, F, E, relu=True, alpha=0.5)
    finally:
        assert lib.ng_tune(b"chan_block", -1) == 0
    for key in ("O", "gradI", "gradF"):
        np.testing.assert_array_equal(blocked[key], plain[key], err_msg="%s %s" % (name, key))
    ref = {"O": rm.conv_fprop_fast(cd, I, F, alpha=0.5, relu=True), "gradI": rm.conv_bprop_fast(cd, F, E, alpha=0.5),
           "gradF": rm.conv_update_fast(cd, I, E, alpha=0.5)}
    _check(cd, blocked, I, F, E, ref, name + " (blocked)")


STRIDED_FIRST_LAYERS = {
    # AlexNet conv1 on the shard of one of 4 / 8 / 16 GPUs (smaller image, same filter geometry)
    "alexnet_conv1_n32": (32, 3, 64, 1, 35, 35, 1, 11, 11, 0, 2, 2, 1, 4, 4),
    "alexnet_conv1_n16": (16, 3, 64, 1, 39, 37, 1, 11, 11, 0, 2, 2, 1, 4, 4),
    "alexnet_conv1_n8": (8, 3, 64, 1, 35, 35, 1, 11, 11, 0, 2, 2, 1, 4, 4),
    # stride 2, 7x7 (a filter that is not a multiple of the stride), odd padding, 4 channels
    "c4_7x7_stride2_n24": (24, 4, 96, 1, 21, 23, 1, 7, 7, 0, 3, 3, 1, 2, 2),
    # stride 3 with a 5x5 filter and no padding: the last window ends before the image does
    "c3_5x5_stride3_n40": (40, 3, 32, 1, 20, 20, 1, 5, 5, 0, 0, 0, 1, 3, 3),
}


@pytest.mark.parametrize("name", sorted(STRIDED_FIRST_LAYERS))
def test_strided_first_layers_of_small_minibatches_run_as_space_to_depth(ng, lib, name):
    """Fewer than 64 images, fewer than 16 channels, stride > 1: the layer is rewritten as a
    unit-stride layer over st*st times the channels (copies of the input and the filters) and runs
    on the tensor-core path; the weight gradient is gathered back into the filter's own shape."""
    import ctypes
    cfg = STRIDED_FIRST_LAYERS[name]
    cd = rm.ConvDims(*cfg)
    I, F, E = _inputs(cd, 1006)
    ref = {"O": rm.conv_fprop_fast(cd, I, F, alpha=0.5, relu=True), "gradF": rm.conv_update_fast(cd, I, E, alpha=0.5)}
    before = ctypes.c_ulonglong(0)
    after = ctypes.c_ulonglong(0)
    assert lib.ng_fallback_launch_count(ctypes.byref(before)) == 0
    got = _run_all(ng, _layer(ng, cfg, "auto"), I, F, E, relu=True, alpha=0.5, ops="fu")
    assert lib.ng_fallback_launch_count(ctypes.byref(after)) == 0
    assert after.value == before.value, "left the tensor-core path"
    _check(cd, got, I, F, E, ref, name)
    # the same through the im2col form it replaces (switch off): same sums, other order
    try:
        assert lib.ng_tune(b"space_to_depth", 0) == 0
        old = _run_all(ng, _layer(ng, cfg, "auto"), I, F, E, relu=True, alpha=0.5, ops="fu")
    finally:
        assert lib.ng_tune(b"space_to_depth", -1) == 0
    _check(cd, old, I, F, E, ref, name + " (im2col)")
    # fp16 weight gradient
    layer = _layer(ng, cfg, "auto")
    dU = ng.empty(layer.dimF)
    ng.update_conv(layer, ng.array(I), ng.array(E), dU, alpha=0.5)
    aU = _abs_terms(cd, I, F, E)[2]
    M, P, Q = cd.MPQ
    assert_close(dU.get(), ref["gradF"], f32_tol(aU, M * P * Q * cd.N) + 2.0 ** -11 * np.abs(ref["gradF"]), name + " fp16 dW")


@pytest.mark.parametrize("name", sorted(SHARDED))
def test_sharded_minibatch_shapes_run_on_the_tensor_core_path(ng, name):
    cfg = SHARDED[name]
    cd = rm.ConvDims(*cfg)
    I, F, E = _inputs(cd, 1004)
    ref = {"O": rm.conv_fprop_fast(cd, I, F, relu=True), "gradI": rm.conv_bprop_fast(cd, F, E),
           "gradF": rm.conv_update_fast(cd, I, E)}
    # guard cells around the outputs: columns of the padded chunk space must not be stored anywhere
    layer = _layer(ng, cfg, "tensor")
    dI, dF, dE = ng.array(I), ng.array(F), ng.array(E)
    pad = 4096
    bufO = ng.empty((layer.sizeO + 2 * pad,))
    bufB = ng.empty((layer.sizeI + 2 * pad,))
    bufO.fill(7.0)
    bufB.fill(7.0)
    dO = bufO[pad:pad + layer.sizeO].reshape(layer.dimO)
    dB = bufB[pad:pad + layer.sizeI].reshape(layer.dimI)
    dU = ng.empty(layer.dimF, dtype=np.float32)
    ng.fprop_conv(layer, dI, dF, dO, relu=True)
    ng.bprop_conv(layer, dF, dE, dB)
    ng.update_conv(layer, dI, dE, dU)
    got = {"O": dO.get(), "gradI": dB.get(), "gradF": dU.get()}
    _check(cd, got, I, F, E, ref, name)
    for buf, size in ((bufO, layer.sizeO), (bufB, layer.sizeI)):
        h = buf.get()
        assert (h[:pad] == 7.0).all() and (h[pad + size:] == 7.0).all(), name + ": wrote outside the tensor"


@pytest.mark.parametrize("name", ["c3_3x3_n64_first_layer", "c3_11x11_stride4_n64_alexnet1", "c64_3x3_n64"])
def test_update_im2col_path(ng, name):
    cfg = CASES[name]
    cd = rm.ConvDims(*cfg)
    I, F, E = _inputs(cd, 77)
    got = _run_all(ng, _layer(ng, cfg, "im2col"), I, F, E, ops="u")
    _check(cd, got, I, F, E, {"gradF": rm.conv_update_fast(cd, I, E)}, name + "/im2col")


def test_shapes_outside_the_tensor_path_run_on_simt(ng):
    cfg = (8, 24, 16, 1, 5, 5, 1, 3, 3, 0, 1, 1, 1, 2, 2)   # N = 8 with a W stride: no 64-element chunks
    cd = rm.ConvDims(*cfg)
    I, F, E = _inputs(cd, 5)
    ref = {"O": rm.conv_fprop(cd, I, F), "gradI": rm.conv_bprop(cd, F, E), "gradF": rm.conv_update(cd, I, E)}
    _check(cd, _run_all(ng, _layer(ng, cfg, "auto"), I, F, E), I, F, E, ref, "auto->simt")
    with pytest.raises(_lib.NervanaError):
        _run_all(ng, _layer(ng, cfg, "tensor"), I, F, E, ops="f")


def test_update_fp16_output_and_determinism(ng):
    cfg = CASES["c64_3x3_n64"]
    cd = rm.ConvDims(*cfg)
    I, F, E = _inputs(cd, 9)
    layer = _layer(ng, cfg)
    dI, dE = ng.array(I), ng.array(E)
    u16 = ng.empty(layer.dimF, dtype=np.float16)
    ng.update_conv(layer, dI, dE, u16)
    ref = rm.conv_update_fast(cd, I, E)
    assert_close(u16.get(), ref, 2.0 ** -10 * np.abs(ref) + 1e-3, "fp16 dW")
    a, b = ng.empty(layer.dimF, dtype=np.float32), ng.empty(layer.dimF, dtype=np.float32)
    ng.update_conv(layer, dI, dE, a)
    ng.update_conv(layer, dI, dE, b)
    assert np.array_equal(a.get(), b.get())     # fixed summation order, unlike atomics


def test_full_size_alexnet_layer_properties(ng):
    """AlexNet conv3 at BASELINE size (N=128, 192->384, 13x13): the oracle is too slow for every
    output, so check (a) linearity in the filter, (b) an exact sample of output pixels."""
    cfg = (128, 192, 384, 1, 13, 13, 1, 3, 3, 0, 1, 1, 1, 1, 1)
    cd = rm.ConvDims(*cfg)
    rng = np.random.default_rng(1003)
    I = rng.uniform(0, 1, cd.dimI).astype(np.float16)
    F1 = (rng.integers(-8, 9, cd.dimF) / 256.0).astype(np.float16)
    F2 = (rng.integers(-8, 9, cd.dimF) / 256.0).astype(np.float16)
    layer = _layer(ng, cfg)
    dI = ng.array(I)
    outs = []
    for F in (F1, F2, (F1 + F2).astype(np.float16)):
        dO = ng.empty(layer.dimO)
        ng.fprop_conv(layer, dI, ng.array(F), dO)
        outs.append(dO.get().astype(np.float32))
    s = outs[0] + outs[1]
    assert (np.abs(outs[2] - s) <= 3 * 2.0 ** -10 * (np.abs(s) + np.abs(outs[0]) + np.abs(outs[1])) + 1e-3).all()
    # exact sample: 6 output pixels through the per-pixel oracle arithmetic
    F2d = F1.astype(np.float32).reshape(-1, cd.K)
    I2 = np.zeros((cd.C * 169 + 1, cd.N), np.float32)
    I2[:-1] = I.astype(np.float32).reshape(-1, cd.N)
    for (p, q) in [(0, 0), (0, 12), (6, 6), (12, 0), (12, 12), (3, 9)]:
        rows = rm._conv_pixel_rows(cd, 0, p - 1, q - 1)
        ref = np.dot(F2d.T, I2[rows, :])
        absd = np.dot(np.abs(F2d).T, np.abs(I2[rows, :]))
        assert_close(outs[0][:, 0, p, q, :], ref, rn16_tol(ref, absd, cd.C * 9), "pixel %d,%d" % (p, q))


FULL_SIZE = {
    # BASELINE configs at their real sizes: (N, C, K, D, H, W, T, R, S, pads, strides)
    "alexnet_conv1_tap_blocks": (128, 3, 64, 1, 224, 224, 1, 11, 11, 0, 2, 2, 1, 4, 4),
    "alexnet_conv2_stacked_update": (128, 64, 192, 1, 27, 27, 1, 5, 5, 0, 2, 2, 1, 1, 1),
    "vgg_conv4_256_rows": (64, 256, 256, 1, 56, 56, 1, 3, 3, 0, 1, 1, 1, 1, 1),
    "config5_3d_conv": (32, 64, 64, 16, 56, 56, 3, 3, 3, 1, 1, 1, 1, 1, 1),
}


@pytest.mark.parametrize("name", sorted(FULL_SIZE))
def test_full_size_adjoint_identity(ng, name):
    """At full size the three passes are checked against each other: they are the three partial
    derivatives of one bilinear form, so <fprop(I, F), E> = <I, bprop(F, E)> = <F, update(I, E)>."""
    cfg = FULL_SIZE[name]
    cd = rm.ConvDims(*cfg)
    rng = np.random.default_rng(1004)
    I = rng.uniform(0, 1, cd.dimI).astype(np.float16)
    F = rng.normal(0, 0.05, cd.dimF).astype(np.float16)
    E = (rng.uniform(-1, 1, cd.dimO) * 0.125).astype(np.float16)
    got = _run_all(ng, _layer(ng, cfg), I, F, E)
    f64 = np.float64
    via_fprop = np.sum(got["O"].astype(f64) * E.astype(f64))
    via_bprop = np.sum(got["gradI"].astype(f64) * I.astype(f64))
    via_update = np.sum(got["gradF"].astype(f64) * F.astype(f64))
    scale = np.sum(np.abs(got["O"].astype(f64)) * np.abs(E.astype(f64)))
    assert np.isfinite([via_fprop, via_bprop, via_update]).all() and scale > 0
    # fp16 rounding of O and gradI: relative 2^-11 per element, random in sign; a dropped tap or a
    # misplaced tile would show at the percent level
    assert abs(via_fprop - via_update) <= 1e-3 * scale, (via_fprop, via_update, scale)
    assert abs(via_fprop - via_bprop) <= 1e-3 * scale, (via_fprop, via_bprop, scale)
    assert abs(via_bprop - via_update) <= 1e-3 * scale, (via_bprop, via_update, scale)


def test_layer_argument_checks(ng):
    with pytest.raises(AssertionError):
        ng.conv_layer(np.float16, 12, 3, 8, 1, 8, 8, 1, 3, 3)       # N % 8
    with pytest.raises(AssertionError):
        ng.conv_layer(np.float16, 16, 3, 12, 1, 8, 8, 1, 3, 3)      # K % 8
    layer = ng.conv_layer(np.float16, 16, 3, 8, 1, 8, 8, 1, 3, 3)
    with pytest.raises(AssertionError):
        ng.fprop_conv(layer, ng.empty((3, 1, 8, 8, 8)), ng.empty(layer.dimF), ng.empty(layer.dimO))   # sizeI
    with pytest.raises(TypeError):
        ng.fprop_conv(layer, ng.empty(layer.dimI, dtype=np.float32), ng.empty(layer.dimF, dtype=np.float32),
                      ng.empty(layer.dimO, dtype=np.float32))
