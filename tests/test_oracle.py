"""The oracle against what the reference itself pins (CPU only).

 * golden vectors: outputs of the reference's own numpy validation code (benchmarks/conv_test.py,
   benchmarks/pool_test.py) captured by tests/golden/make_golden.py;
 * known-answer cases of the reference's tests: all-ones GEMM == k, zeros == 0
   (kernels/C_interface/test.cu:27-55,70; benchmarks/gemm_test2.py:30-43), ones convolution
   (benchmarks/conv_test.py:58-61);
 * the unit-test recipe for element-wise results (nervanagpu/tests/test_tensor.py:46-57).
"""
import numpy as np
import pytest

from oracle import reference_math as rm
from tests._util import golden, golden_names


@pytest.mark.parametrize("name", golden_names("conv_"))
def test_conv_oracle_matches_reference_numpy_path(name):
    g = golden(name)
    cd = rm.ConvDims(*[int(v) for v in g["cfg"]])
    # same loop, same association order: identical fp32 results
    np.testing.assert_array_equal(rm.conv_fprop(cd, g["I"], g["F"]), g["O"])
    np.testing.assert_array_equal(rm.conv_update(cd, g["I"], g["E"]), g["gradF"])
    np.testing.assert_allclose(rm.conv_bprop(cd, g["F"], g["E"]), g["gradI"], rtol=0, atol=1e-4)
    # vectorised variants: same sums, other order
    scale = np.abs(g["O"]).max()
    np.testing.assert_allclose(rm.conv_fprop_fast(cd, g["I"], g["F"]), g["O"], rtol=0, atol=1e-5 * scale)
    np.testing.assert_allclose(rm.conv_bprop_fast(cd, g["F"], g["E"]), g["gradI"], rtol=0,
                               atol=1e-5 * np.abs(g["gradI"]).max())
    np.testing.assert_allclose(rm.conv_update_fast(cd, g["I"], g["E"]), g["gradF"], rtol=0,
                               atol=1e-5 * np.abs(g["gradF"]).max())


@pytest.mark.parametrize("name", golden_names("pool_"))
def test_pool_oracle_matches_reference_numpy_path(name):
    g = golden(name)
    pd = rm.PoolDims(*[int(v) for v in g["cfg"]])
    O, gradI = rm.pool_max(pd, g["I"], E=g["O"])
    np.testing.assert_array_equal(O, g["O"])
    np.testing.assert_array_equal(gradI, g["gradI"])


@pytest.mark.parametrize("size", [257, 256, 255, 129, 128, 127, 65, 64, 17, 16, 15])
@pytest.mark.parametrize("op", ["nn", "nt", "tn"])
def test_gemm_known_answers(size, op):
    ones = np.ones((size, size), dtype=np.float16)
    C = rm.gemm(ones, ones, a_t=op[0] == "t", b_t=op[1] == "t")
    assert (C == size).all()
    zeros = np.zeros((size, size), dtype=np.float16)
    assert (rm.gemm(zeros, zeros, a_t=op[0] == "t", b_t=op[1] == "t") == 0).all()


def test_gemm_epilogue_order():
    A = np.array([[1.0, -2.0]], dtype=np.float16)
    B = np.array([[3.0], [1.0]], dtype=np.float16)
    C = np.array([[10.0]], dtype=np.float16)
    # acc = 1 -> alpha -> relu -> + beta*C : relu acts before the beta term
    assert rm.gemm(A, B, alpha=-1.0, beta=0.5, relu=True, C=C)[0, 0] == 5.0
    assert rm.gemm(A, B, alpha=2.0, beta=0.5, relu=True, C=C)[0, 0] == 7.0


def test_conv_ones_known_answer():
    cd = rm.ConvDims(8, 3, 8, 1, 6, 6, 1, 3, 3, 0, 1, 1, 1, 1, 1)
    O = rm.conv_fprop(cd, np.ones(cd.dimI, np.float32), np.ones(cd.dimF, np.float32))
    # interior pixels see all 27 taps, corners 12
    assert O[0, 0, 2, 2, 0] == 27 and O[0, 0, 0, 0, 0] == 12
    assert cd.MPQ == (1, 6, 6)


def test_layer_dims_formula():
    # AlexNet conv1: (224 - 11 + 1 + 4) / 4 = 54.5 -> 55 (nervanagpu/layers.py:297-301)
    cd = rm.ConvDims(128, 3, 64, 1, 224, 224, 1, 11, 11, 0, 2, 2, 1, 4, 4)
    assert cd.MPQ == (1, 55, 55)
    pd = rm.PoolDims(128, 64, 1, 55, 55, 1, 1, 3, 3, 0, 0, 0, 0, 1, 1, 2, 2)
    assert (pd.K,) + pd.MPQ == (64, 1, 27, 27)


def test_pool_first_maximum_wins():
    pd = rm.PoolDims(1, 1, 1, 2, 2, 1, 1, 2, 2)
    I = np.full(pd.dimI, 3.0, dtype=np.float32)
    O, gradI = rm.pool_max(pd, I, E=np.full(pd.dimO, 7.0, np.float32))
    assert O.ravel()[0] == 3.0
    assert gradI.ravel().tolist() == [7.0, 0.0, 0.0, 0.0]


def test_cast_recipe_of_reference_unit_test():
    x = np.array([-300.4, -0.5, 0.5, 1.5, 2.5, 126.6, 300.0], dtype=np.float32)
    assert rm.cast_result(x, np.int8).tolist() == [-128, 0, 0, 2, 2, 127, 127]
    assert rm.cast_result(x, np.uint8).tolist() == [0, 0, 0, 2, 2, 127, 255]
    assert rm.cast_result(np.float32(0.1) + np.float32(0.2), np.float16) == np.float16(np.float32(0.1) + np.float32(0.2))


def test_batch_norm_expression():
    rng = np.random.default_rng(1005)
    A = rng.uniform(0, 1, (64, 128)).astype(np.float16)
    out = rm.batch_norm(A)
    assert abs(out.mean(axis=1)).max() < 1e-5
    assert abs(out.var(axis=1) - 1).max() < 0.02   # eps = 1e-3 on a variance of ~1/12


def test_fp16_neighbours():
    x = np.array([1.0, 1.0 + 2.0 ** -11, -(1.0 + 2.0 ** -11), 3e-6, 70000.0, 0.0], dtype=np.float32)
    lo, hi = rm.fp16_neighbours(x)
    assert lo[0] == hi[0] == np.float16(1.0)
    assert lo[1] == np.float16(1.0) and hi[1] == np.float16(1.0 + 2.0 ** -10)
    assert lo[2] == np.float16(-1.0) and hi[2] == np.float16(-(1.0 + 2.0 ** -10))
    assert float(lo[3]) <= 3e-6 <= float(hi[3]) and float(hi[3]) - float(lo[3]) == 2.0 ** -24
    assert lo[4] == hi[4] == np.float16(65504.0)
    assert lo[5] == hi[5] == 0


@pytest.mark.parametrize("op", ["avg", "l2"])
def test_pool_avg_l2_oracle_follows_the_reference_numpy_definition(op):
    """benchmarks/pool_test.py:141-146: mean / root-sum-square over all window positions, the
    positions outside the tensor reading zeros. Checked against plain loops on a padded case."""
    pd = rm.PoolDims(4, 3, 1, 5, 5, 1, 1, 3, 3, 0, 0, 1, 1, 1, 1, 2, 2)
    rng = np.random.default_rng(5)
    I = rng.uniform(-1, 1, pd.dimI).astype(np.float32)
    E = rng.uniform(-1, 1, pd.dimO).astype(np.float32)
    O, gradI = rm.pool_avg_l2(pd, I, op, E)
    M, P, Q = pd.MPQ
    want = np.zeros(pd.dimO, np.float32)
    grad = np.zeros(pd.dimI, np.float32)
    for k in range(pd.K):
        for p in range(P):
            for q in range(Q):
                pos = [(k, 0, p * 2 - 1 + r, q * 2 - 1 + s) for r in range(3) for s in range(3)]
                vals = [I[c, z, y, x, :] if 0 <= y < 5 and 0 <= x < 5 else np.zeros(4, np.float32)
                        for (c, z, y, x) in pos]
                if op == "avg":
                    want[k, 0, p, q] = sum(vals) / 9.0
                else:
                    want[k, 0, p, q] = np.sqrt(sum(v * v for v in vals))
                norm = want[k, 0, p, q].astype(np.float16).astype(np.float32)
                for (c, z, y, x), v in zip(pos, vals):
                    if 0 <= y < 5 and 0 <= x < 5:
                        if op == "avg":
                            grad[c, z, y, x] += E[k, 0, p, q] / 9.0
                        else:
                            grad[c, z, y, x] += np.where(norm > 0, E[k, 0, p, q] * v / np.where(norm > 0, norm, 1), 0)
    assert np.allclose(O, want, rtol=1e-6, atol=1e-7)
    assert np.allclose(gradI, grad, rtol=1e-5, atol=1e-6)


SAMPLED_CONV = [(16, 5, 8, 1, 9, 7, 1, 3, 3, 0, 1, 1, 1, 2, 1), (8, 4, 8, 4, 6, 6, 3, 3, 3, 1, 1, 1, 1, 1, 1),
                (8, 3, 8, 1, 23, 23, 1, 11, 11, 0, 2, 2, 1, 4, 4)]


@pytest.mark.parametrize("cfg", SAMPLED_CONV)
def test_sampled_conv_oracle_equals_the_loop_form(cfg):
    """The per-position functions used at full size against the loops of conv_test.py:147-167."""
    cd = rm.ConvDims(*cfg)
    rng = np.random.default_rng(3)
    I = rng.uniform(0, 1, cd.dimI).astype(np.float16)
    F = rng.normal(0, 0.1, cd.dimF).astype(np.float16)
    E = rng.uniform(-1, 1, cd.dimO).astype(np.float16)
    (M, P, Q), (D, H, W), (T, R, S) = cd.MPQ, cd.DHW, cd.TRS
    pix = [(0, 0, 0), (M - 1, P - 1, Q - 1), (M // 2, P // 2, Q // 2)]
    for m, p, q in pix:
        args = (cd, m * cd.strides[0] - cd.padding[0], p * cd.strides[1] - cd.padding[1],
                q * cd.strides[2] - cd.padding[2])
        assert list(rm.conv_pixel_rows_np(*args)) == rm._conv_pixel_rows(*args)
    O = rm.conv_fprop(cd, I, F)
    for got, (m, p, q) in zip(rm.conv_fprop_pixels(cd, I, F, pix), pix):
        np.testing.assert_array_equal(got, O[:, m, p, q, :])
    B = rm.conv_bprop(cd, F, E)
    pos = [(0, 0, 0), (D - 1, H - 1, W - 1), (D // 2, H // 2, W // 3), (0, 1, 2)]
    for got, (z, y, x) in zip(rm.conv_bprop_pixels(cd, F, E, pos), pos):
        np.testing.assert_allclose(got, B[:, z, y, x, :], rtol=0, atol=1e-4)
    U = rm.conv_update(cd, I, E)
    taps = [(0, 0, 0), (T - 1, R - 1, S - 1), (T // 2, R // 2, S // 2)]
    for got, (t, r, s) in zip(rm.conv_update_taps(cd, I, E, taps), taps):
        np.testing.assert_allclose(got, U[:, t, r, s, :], rtol=1e-5, atol=1e-4)


@pytest.mark.parametrize("cfg", [(16, 8, 1, 13, 13, 1, 1, 3, 3, 0, 0, 0, 0, 1, 1, 2, 2),
                                 (8, 8, 4, 6, 6, 2, 2, 2, 2, 0, 0, 0, 0, 2, 2, 2, 2),
                                 (16, 5, 1, 9, 9, 1, 1, 3, 3, 0, 0, 1, 1, 1, 1, 2, 2),
                                 (8, 2, 1, 9, 9, 1, 1, 2, 2, 0, 0, 0, 0, 1, 1, 3, 3)])
def test_fast_pool_oracle_is_bit_identical_to_the_loop_form(cfg):
    pd = rm.PoolDims(*cfg)
    rng = np.random.default_rng(4)
    I = (rng.integers(0, 12, pd.dimI) / 8.0).astype(np.float16)      # many ties
    E = rng.uniform(-1, 1, pd.dimO).astype(np.float16)
    O, B = rm.pool_max(pd, I, E)
    O2, B2 = rm.pool_max_fast(pd, I, E)
    np.testing.assert_array_equal(O, O2)
    np.testing.assert_array_equal(B, B2)
