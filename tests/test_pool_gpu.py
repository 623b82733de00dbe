"""fprop_pool / bprop_pool: bit-exact against the reference's numpy path (B200 only)."""
import numpy as np
import pytest

from oracle import reference_math as rm
from tests._util import golden, golden_names

pytestmark = pytest.mark.gpu


def _run(ng, cfg, I, E, dtype=np.float16):
    layer = ng.pool_layer(dtype, "max", *cfg)
    dI, dE = ng.array(I, dtype=dtype), ng.array(E, dtype=dtype)
    dO, dB = ng.empty(layer.dimO, dtype=dtype), ng.empty(layer.dimI, dtype=dtype)
    ng.fprop_pool(layer, dI, dO)
    ng.bprop_pool(layer, dI, dE, dB)
    return layer, dO.get(), dB.get()


@pytest.mark.parametrize("name", golden_names("pool_"))
def test_golden_vectors_of_the_reference_numpy_path(ng, name):
    g = golden(name)
    cfg = [int(v) for v in g["cfg"]]
    # the reference script back-propagates its own output
    layer, O, B = _run(ng, cfg, g["I"], g["O"].astype(np.float16))
    assert np.array_equal(O.astype(np.float32), g["O"])
    assert np.array_equal(B, g["gradI"].astype(np.float16))


CASES = {
    # (N, C, D, H, W, J, T, R, S, pad_j, pad_d, pad_h, pad_w, str_j, str_d, str_h, str_w)
    "alexnet_3x3_s2_n64": (64, 8, 1, 13, 13, 1, 1, 3, 3, 0, 0, 0, 0, 1, 1, 2, 2),
    "vgg_2x2_n32": (32, 8, 1, 8, 8, 1, 1, 2, 2, 0, 0, 0, 0, 1, 1, 2, 2),
    "config5_jtrs_2222": (32, 8, 4, 6, 6, 2, 2, 2, 2, 0, 0, 0, 0, 2, 2, 2, 2),
    "padded_overlapping": (16, 5, 1, 9, 9, 2, 1, 3, 3, 1, 0, 1, 1, 1, 1, 2, 2),
    "n4_scalar_lanes": (4, 3, 1, 7, 7, 1, 1, 3, 3, 0, 0, 0, 0, 1, 1, 2, 2),
    "stride_larger_than_window": (8, 2, 1, 9, 9, 1, 1, 2, 2, 0, 0, 0, 0, 1, 1, 3, 3),
    "maxout_over_feature_maps": (64, 16, 1, 1, 1, 4, 1, 1, 1, 0, 0, 0, 0, 4, 1, 1, 1),
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_bit_exact_against_oracle(ng, name):
    cfg = CASES[name]
    pd = rm.PoolDims(*cfg)
    rng = np.random.default_rng(1005)
    # few distinct values: plenty of ties, so the first-maximum rule is exercised
    I = (rng.integers(0, 12, pd.dimI) / 8.0).astype(np.float16)
    E = rng.uniform(-1, 1, pd.dimO).astype(np.float16)
    refO, refB = rm.pool_max(pd, I, E)
    layer, O, B = _run(ng, cfg, I, E)
    assert layer.dimO == pd.dimO
    assert np.array_equal(O, refO.astype(np.float16))
    assert np.array_equal(B, refB.astype(np.float16))


@pytest.mark.parametrize("name", sorted(CASES))
def test_fused_relu_mask_equals_bprop_then_mask(ng, name):
    cfg = CASES[name]
    pd = rm.PoolDims(*cfg)
    rng = np.random.default_rng(31)
    # a ReLU output: about half zeros (whole windows of zeros included), ties among the rest
    I = (np.maximum(rng.integers(-8, 6, pd.dimI), 0) / 4.0).astype(np.float16)
    E = rng.uniform(-1, 1, pd.dimO).astype(np.float16)
    _, refB = rm.pool_max(pd, I, E)
    ref = (refB * (I > 0)).astype(np.float16)           # Layer.bprop_relu on the pool's deltas
    layer = ng.pool_layer(np.float16, "max", *cfg)
    dI, dE, dB = ng.array(I), ng.array(E), ng.empty(layer.dimI)
    ng.bprop_pool(layer, dI, dE, dB, relu_mask=True)
    assert np.array_equal(dB.get(), ref)
    assert (ref != refB.astype(np.float16)).any() or not (I[refB != 0] <= 0).any()


@pytest.mark.parametrize("name", ["alexnet_3x3_s2_n64", "vgg_2x2_n32", "stride_larger_than_window"])
@pytest.mark.parametrize("mask", [False, True])
def test_recorded_argmax_gives_the_same_backward_pass(ng, name, mask):
    cfg = CASES[name]
    pd = rm.PoolDims(*cfg)
    rng = np.random.default_rng(77)
    I = (np.maximum(rng.integers(-8, 6, pd.dimI), 0) / 4.0).astype(np.float16)
    E = rng.uniform(-1, 1, pd.dimO).astype(np.float16)
    layer = ng.pool_layer(np.float16, "max", *cfg)
    nbytes = ng.pool_argmax_bytes(layer)
    if name == "stride_larger_than_window":
        assert nbytes == 0                      # no specialised path: callers fall back
        return
    assert nbytes == int(np.prod(pd.dimO))
    dI, dE = ng.array(I), ng.array(E)
    O1, O2 = ng.empty(layer.dimO), ng.empty(layer.dimO)
    B1, B2 = ng.empty(layer.dimI), ng.empty(layer.dimI)
    rec = ng.empty((nbytes,), dtype=np.uint8)
    ng.fprop_pool(layer, dI, O1)
    ng.fprop_pool(layer, dI, O2, argmax=rec)
    ng.bprop_pool(layer, dI, dE, B1, relu_mask=mask)
    dI.fill(0)                                  # the recorded pass must not need the input
    ng.bprop_pool(layer, dI, dE, B2, relu_mask=mask, argmax=rec)
    assert np.array_equal(O1.get(), O2.get())
    assert np.array_equal(B1.get(), B2.get())


def test_fp32_pooling(ng):
    cfg = CASES["alexnet_3x3_s2_n64"]
    pd = rm.PoolDims(*cfg)
    rng = np.random.default_rng(2)
    I = rng.uniform(0, 1, pd.dimI).astype(np.float32)
    E = rng.uniform(-1, 1, pd.dimO).astype(np.float32)
    refO, refB = rm.pool_max(pd, I, E)
    _, O, B = _run(ng, cfg, I, E, dtype=np.float32)
    assert np.array_equal(O, refO)
    assert np.array_equal(B, refB)


def test_full_size_alexnet_pool1_properties(ng):
    """pool1 at BASELINE size (N=128, C=64, 55x55 -> 27x27, 3x3 stride 2): size-independent checks.
    Every output is >= each tap of its window and equals one of them; bprop conserves the sum of E
    (each error lands on exactly one input) and puts nothing where the input is not a window max."""
    cfg = (128, 64, 1, 55, 55, 1, 1, 3, 3, 0, 0, 0, 0, 1, 1, 2, 2)
    pd = rm.PoolDims(*cfg)
    rng = np.random.default_rng(1003)
    I = rng.uniform(0, 1, pd.dimI).astype(np.float16)
    E = (rng.integers(1, 5, pd.dimO) / 4.0).astype(np.float16)
    _, O, B = _run(ng, cfg, I, E)
    taps = np.stack([I[:, :, r:r + 53:2, s:s + 53:2, :] for r in range(3) for s in range(3)])
    assert np.array_equal(O, taps.max(axis=0))
    assert abs(float(B.astype(np.float64).sum()) - float(E.astype(np.float64).sum())) <= 1e-6 * E.size
    assert (B >= 0).all() and (B[:, :, 55 - 0:, :, :] == 0).all()
    # sampled channels against the oracle, bit for bit
    sub = rm.PoolDims(128, 2, 1, 55, 55, 1, 1, 3, 3, 0, 0, 0, 0, 1, 1, 2, 2)
    refO, refB = rm.pool_max(sub, I[5:7], E[5:7])
    assert np.array_equal(O[5:7], refO.astype(np.float16))
    assert np.array_equal(B[5:7], refB.astype(np.float16))


@pytest.mark.parametrize("op", ["avg", "l2"])
@pytest.mark.parametrize("name", sorted(CASES))
def test_avg_and_l2_pooling_against_oracle(ng, name, op):
    """The ops the reference defines in numpy only (benchmarks/pool_test.py:141-146). Forward: the
    fp32 result rounded to fp16 (one ulp of slack for the order of the fp32 additions); backward:
    the derivative of the forward definition, tolerance 2 fp16 ulps of the largest term sum."""
    cfg = CASES[name]
    pd = rm.PoolDims(*cfg)
    rng = np.random.default_rng(77)
    I = rng.uniform(-1, 1, pd.dimI).astype(np.float16)
    E = rng.uniform(-1, 1, pd.dimO).astype(np.float16)
    refO, refB = rm.pool_avg_l2(pd, I, op, E)
    layer = ng.pool_layer(np.float16, op, *cfg)
    dI, dE = ng.array(I), ng.array(E)
    dO, dB = ng.empty(layer.dimO), ng.empty(layer.dimI)
    ng.fprop_pool(layer, dI, dO)
    ng.bprop_pool(layer, dI, dE, dB)
    O, B = dO.get().astype(np.float32), dB.get().astype(np.float32)
    assert np.all(np.abs(O - refO) <= 2.0 ** -10 * np.maximum(np.abs(refO), 2.0 ** -14))
    windows = np.prod(pd.JTRS)
    assert np.all(np.abs(B - refB) <= 2.0 ** -9 * np.maximum(np.abs(refB), 1.0) * max(1, windows // 4))
    assert np.abs(B).sum() > 0


def test_avg_and_l2_refuse_the_max_only_extensions(ng):
    cfg = CASES["vgg_2x2_n32"]
    layer = ng.pool_layer(np.float16, "avg", *cfg)
    dI, dE, dB = ng.empty(layer.dimI), ng.empty(layer.dimO), ng.empty(layer.dimI)
    with pytest.raises(ValueError):
        ng.bprop_pool(layer, dI, dE, dB, relu_mask=True)
