"""Generated element-wise / reduction kernels and stochastic rounding on the device (B200 only).

The first test is the reference's only unit test restated (nervanagpu/tests/test_tensor.py:46-82):
results computed by numpy in fp32, integers rounded + clipped, cast, compared with atol 1e-5.
"""
import numpy as np
import pytest

from oracle import reference_math as rm

pytestmark = pytest.mark.gpu


def _rand_unif(rng, dtype, dims):
    if np.dtype(dtype).kind == "f":
        return rng.uniform(-1, 1, dims).astype(dtype)
    info = np.iinfo(dtype)
    return np.around(rng.uniform(info.min, info.max, dims)).clip(info.min, info.max)


_BINARY = {
    "+": lambda a, b: a + b, "-": lambda a, b: a - b, "*": lambda a, b: a * b,
    ">": lambda a, b: a > b, ">=": lambda a, b: a >= b, "<": lambda a, b: a < b, "<=": lambda a, b: a <= b,
}


@pytest.mark.parametrize("dtype", [np.float32, np.float16, np.int8, np.uint8])
def test_math_like_the_reference_unit_test(ng, dtype):
    rng = np.random.default_rng(42)
    dims = (1024, 1024)
    inA, inB = _rand_unif(rng, dtype, dims), _rand_unif(rng, dtype, dims)
    A, B, C = ng.array(inA, dtype=dtype), ng.array(inB, dtype=dtype), ng.empty(dims, dtype=dtype)
    hA, hB = A.get().astype(np.float32), B.get().astype(np.float32)
    for sym, fn in _BINARY.items():
        C[:] = fn(A, B)
        ref = rm.cast_result(np.asarray(fn(hA, hB), dtype=np.float32), dtype)
        np.testing.assert_allclose(C.get().astype(np.float32), ref.astype(np.float32), rtol=0, atol=1e-5, err_msg=sym)


def test_division_and_transcendentals(ng):
    rng = np.random.default_rng(1)
    a = rng.uniform(0.5, 2.0, (256, 512)).astype(np.float32)
    b = rng.uniform(0.5, 2.0, (256, 512)).astype(np.float32)
    A, B, C = ng.array(a, dtype=np.float32), ng.array(b, dtype=np.float32), ng.empty(a.shape, dtype=np.float32)
    C[:] = A / B
    np.testing.assert_array_equal(C.get(), a / b)           # IEEE division, no fast-math
    C[:] = ng.sqrt(A) + ng.exp(-B) * ng.log(A) + ng.tanh(B) + ng.sig(A) + ng.power(A, 2.0)
    ref = np.sqrt(a) + np.exp(-b) * np.log(a) + np.tanh(b) + 1 / (1 + np.exp(-a)) + a ** 2
    np.testing.assert_allclose(C.get(), ref, rtol=2e-6, atol=1e-6)
    C[:] = ng.clip(A - B, -0.25, 0.25) + ng.maximum(A, B) * ng.minimum(A, 1.0) + abs(A - B) - (-A)
    ref = np.clip(a - b, -0.25, 0.25) + np.maximum(a, b) * np.minimum(a, 1.0) + abs(a - b) + a
    np.testing.assert_allclose(C.get(), ref, rtol=1e-6, atol=1e-6)


def test_scalar_assign_views_broadcast_transpose(ng):
    rng = np.random.default_rng(2)
    a = rng.uniform(-1, 1, (96, 200)).astype(np.float16)
    A = ng.array(a)
    C = ng.zeros((96, 200))
    assert (C.get() == 0).all()
    C.fill(1.5)
    assert (C.get() == 1.5).all()
    C[8:24, 16:48] = 3                      # strided view: generated kernel, not memset
    ref = np.full((96, 200), 1.5, np.float16)
    ref[8:24, 16:48] = 3
    assert np.array_equal(C.get(), ref)
    col = ng.array(a[:, :1].copy())
    row = ng.array(a[:1, :].copy())
    C[:] = A * col + row
    ref = (a.astype(np.float32) * a[:, :1].astype(np.float32) + a[:1, :].astype(np.float32)).astype(np.float16)
    assert np.array_equal(C.get(), ref)
    Ct = ng.empty((200, 96))
    Ct[:] = A.T
    assert np.array_equal(Ct.get(), a.T)
    D = ng.empty((96, 200))
    D[:] = A                                 # contiguous same dtype: device copy
    assert np.array_equal(D.get(), a)
    F32 = ng.empty((96, 200), dtype=np.float32)
    F32[:] = A                               # dtype conversion
    assert np.array_equal(F32.get(), a.astype(np.float32))


@pytest.mark.parametrize("shape", [(4096, 128), (37, 1000), (16, 5000)])
def test_reductions_both_axes(ng, shape):
    rng = np.random.default_rng(3)
    a = rng.uniform(-1, 1, shape).astype(np.float16)
    A = ng.array(a)
    af = a.astype(np.float32)
    for axis in (0, 1):
        oshape = (1, shape[1]) if axis == 0 else (shape[0], 1)
        out = ng.empty(oshape, dtype=np.float32)
        ng.sum(A, axis=axis, out=out)
        np.testing.assert_allclose(out.get(), af.sum(axis=axis, keepdims=True), rtol=1e-5, atol=1e-3)
        ng.max(A, axis=axis, out=out)
        assert np.array_equal(out.get(), af.max(axis=axis, keepdims=True))
        ng.min(A, axis=axis, out=out)
        assert np.array_equal(out.get(), af.min(axis=axis, keepdims=True))
        idx = ng.empty(oshape, dtype=np.int32)
        ng.argmax(A, axis=axis, out=idx)
        assert np.array_equal(idx.get(), af.argmax(axis=axis).reshape(oshape))
        ng.argmin(A, axis=axis, out=idx)
        assert np.array_equal(idx.get(), af.argmin(axis=axis).reshape(oshape))
    part = ng.empty((shape[0], 1), dtype=np.float32)
    total = ng.empty((1, 1), dtype=np.float32)
    ng.sum(A, partial=part, out=total)
    np.testing.assert_allclose(total.get()[0, 0], af.sum(dtype=np.float64), rtol=1e-4, atol=1e-2)
    ng.mean(abs(A), partial=part, out=part[0:1, 0:1])
    np.testing.assert_allclose(part.get()[0, 0], np.abs(af).mean(dtype=np.float64), rtol=1e-4)


def test_config5_batch_norm_expression(ng):
    """BASELINE config 5: (A - mean(A,axis=1)) / sqrt(var(A,axis=1) + 1e-3) on 4096x128 fp16 U(0,1).
    Tolerance: one fp16 ulp of the fp32 numpy result."""
    rng = np.random.default_rng(1005)
    a = rng.uniform(0, 1, (4096, 128)).astype(np.float16)
    A = ng.array(a)
    A[:] = (A - ng.mean(A, axis=1)) / ng.sqrt(ng.var(A, axis=1) + 1e-3)
    ref = rm.batch_norm(a, eps=1e-3, axis=1)
    got = A.get().astype(np.float32)
    ulp = np.maximum(2.0 ** (np.floor(np.log2(np.maximum(np.abs(ref), 2.0 ** -14))) - 10), 2.0 ** -24)
    # one fp16 ulp, plus the fp32 summation-order slack of a 128-term mean/variance (matters only
    # for outputs next to zero, whose fp16 ulp is smaller than fp32 rounding of the inputs' mean)
    assert (np.abs(got - ref) <= ulp + 4e-6).all()
    # axis 0 variant into a separate output
    B = ng.array(a)
    O = ng.empty(a.shape, dtype=np.float32)
    O[:] = (B - ng.mean(B, axis=0)) / ng.sqrt(ng.var(B, axis=0) + 1e-3)
    np.testing.assert_allclose(O.get(), rm.batch_norm(a, eps=1e-3, axis=0), rtol=2e-5, atol=2e-5)


def test_take_onehot_dropout(ng):
    rng = np.random.default_rng(4)
    a = rng.uniform(-1, 1, (50, 64)).astype(np.float16)
    A = ng.array(a)
    rows = rng.integers(0, 50, 20).astype(np.int32)
    out = ng.empty((20, 64))
    out[:] = A.take(ng.array(rows, dtype=np.int32), 0) * 2
    assert np.array_equal(out.get(), (a[rows].astype(np.float32) * 2).astype(np.float16))
    cols = rng.integers(0, 64, 10).astype(np.int32)
    outc = ng.empty((50, 10))
    ng.take(A, ng.array(cols, dtype=np.int32), 1, out=outc)
    assert np.array_equal(outc.get(), a[:, cols])
    labels = rng.integers(0, 10, 64).astype(np.int32)
    hot = ng.empty((10, 64))
    ng.onehot(ng.array(labels, dtype=np.int32), axis=0, out=hot)
    assert np.array_equal(hot.get(), (np.arange(10)[:, None] == labels[None, :]).astype(np.float16))
    mask = ng.empty((512, 512), dtype=np.float32)
    ng.dropout(keep=0.3, out=mask)
    m = mask.get()
    assert set(np.unique(m).tolist()) <= {0.0, 1.0}
    assert abs(m.mean() - 0.3) < 0.01
    u = ng.empty((512, 512), dtype=np.float32)
    ng.rand(out=u)
    h = u.get()
    assert 0.0 <= h.min() and h.max() < 1.0 and abs(h.mean() - 0.5) < 0.01


def test_layer_helpers_relu_mask_and_sgd(ng):
    """bprop_relu (deltas *= activations > 0) and grad_descent (weights += updates * lr), the
    element-wise kernels of the benchmark loop (nervanagpu/layers.py:87-96)."""
    rng = np.random.default_rng(5)
    act = rng.uniform(-1, 1, (256, 64)).astype(np.float16)
    delta = rng.uniform(-1, 1, (256, 64)).astype(np.float16)
    D, Aact = ng.array(delta), ng.array(act)
    D *= Aact > 0
    assert np.array_equal(D.get(), (delta * (act > 0)).astype(np.float16))
    w = rng.normal(0, 0.1, (256, 64)).astype(np.float16)
    u = rng.normal(0, 1, (256, 64)).astype(np.float32)
    W, U = ng.array(w), ng.array(u, dtype=np.float32)
    W += U * 0.01
    ref = (w.astype(np.float32) + u * np.float32(0.01)).astype(np.float16)
    assert np.array_equal(W.get(), ref)


# ---------------------------------------------------------------------------------------------
# stochastic rounding
# ---------------------------------------------------------------------------------------------
def test_stochastic_rounding_elementwise(ng):
    from nervanagpu_b200 import NervanaGPU
    sr = NervanaGPU(stochastic_round=True, seed=1234)
    rng = np.random.default_rng(6)
    x = rng.uniform(-4, 4, (256, 256)).astype(np.float32)
    x[0, :8] = [0.0, 1.0, -1.0, 3e-6, -3e-6, 1e-7, 6e4, -2.0 ** -14]
    X = sr.array(x, dtype=np.float32)
    lo, hi = rm.fp16_neighbours(x)
    R = 64
    acc = np.zeros(x.shape, np.float64)
    first = None
    for r in range(R):
        H = sr.empty(x.shape)                      # fp16, rounding = 10 bits
        H[:] = X * 1
        h = H.get()
        assert ((h == lo) | (h == hi)).all()       # always one of the two neighbours
        acc += h.astype(np.float64)
        first = h if first is None else first
    mean_err = acc / R - x
    ulp = np.abs(hi.astype(np.float64) - lo.astype(np.float64))
    # per element: |mean error| <= 4 sigma, sigma <= ulp / (2 sqrt(R))
    assert (np.abs(mean_err) <= 4 * ulp / (2 * np.sqrt(R)) + 1e-12).all()
    # overall unbiased: z-score of the summed normalised error
    z = (mean_err[ulp > 0] / ulp[ulp > 0]).sum() / np.sqrt((ulp > 0).sum() / (12.0 * R))
    assert abs(z) < 5
    # same seed and offsets: bit-identical rerun
    sr2 = NervanaGPU(stochastic_round=True, seed=1234)
    H2 = sr2.empty(x.shape)
    H2[:] = sr2.array(x, dtype=np.float32) * 1
    assert np.array_equal(H2.get(), first)


def test_stochastic_rounding_gemm(ng):
    """Config 2 with stochastic rounding: each output is a neighbour of the fp32 value (taken from
    the SIMT path's fp32 accumulation order is not needed: neighbours are computed from the oracle
    and widened by the accumulation tolerance), the mean over draws converges, reruns repeat."""
    from nervanagpu_b200 import NervanaGPU
    sr = NervanaGPU(stochastic_round=True, seed=0xB200)
    rng = np.random.default_rng(1002)
    m, n, k = 256, 128, 512
    A = rng.normal(0, 0.1, (m, k)).astype(np.float16)
    B = rng.normal(0, 0.1, (k, n)).astype(np.float16)
    ref = rm.gemm(A, B)
    dA, dB = sr.array(A), sr.array(B)
    R = 48
    acc = np.zeros((m, n), np.float64)
    outs = []
    for r in range(R):
        C = sr.empty((m, n))
        sr.dot(dA, dB, C)
        c = C.get()
        outs.append(c)
        acc += c.astype(np.float64)
    eps = k * 2.0 ** -24 * rm.gemm_abs(A, B)       # fp32 accumulation-order slack
    lo_a, _ = rm.fp16_neighbours(ref - np.sign(ref) * eps)
    _, hi_b = rm.fp16_neighbours(ref + np.sign(ref) * eps)
    lo = np.minimum(lo_a.astype(np.float32), hi_b.astype(np.float32))
    hi = np.maximum(lo_a.astype(np.float32), hi_b.astype(np.float32))
    for c in outs:
        cf = c.astype(np.float32)
        assert ((cf >= lo) & (cf <= hi)).all()
    assert any(not np.array_equal(outs[0], o) for o in outs[1:])      # draws differ
    ulp = np.maximum(2.0 ** (np.floor(np.log2(np.maximum(np.abs(ref), 2.0 ** -14))) - 10), 2.0 ** -24)
    mean_err = acc / R - ref
    assert (np.abs(mean_err) <= 4 * ulp / (2 * np.sqrt(R)) + eps + 1e-9).all()
    z = (mean_err / ulp).sum() / np.sqrt(mean_err.size / (12.0 * R))
    assert abs(z) < 6
    # explicit kwarg overrides the tensor's rounding; offset 0 of a fresh backend repeats draw 0
    sr2 = NervanaGPU(stochastic_round=False, seed=0xB200)
    C2 = sr2.empty((m, n))
    sr2.dot(sr2.array(A), sr2.array(B), C2, stochastic_round=True)
    assert np.array_equal(C2.get(), outs[0])
    C3 = sr.empty((m, n))
    sr.dot(dA, dB, C3, stochastic_round=0)
    assert np.array_equal(C3.get(), ref.astype(np.float16)) or \
        (np.abs(C3.get().astype(np.float32) - ref) <= 2.0 ** -10 * np.abs(ref) + eps).all()


def _kahan_model(s, c, a, cmp_scale, add_scale):
    """numpy restatement of the reference's compensated_sum kernel (nervanagpu/float_ew.py:1430-1482):
    every intermediate in fp32, the new sum and the new compensation rounded to the storage type."""
    f32 = np.float32
    s32, c32, a32 = s.astype(f32), c.astype(f32), a.astype(f32)
    y = a32 * f32(add_scale) - c32 * f32(cmp_scale)
    t = (s32 + y).astype(s.dtype)
    c_new = ((t.astype(f32) - s32) - y).astype(s.dtype)
    return t, c_new


@pytest.mark.parametrize("dtype", [np.float16, np.float32])
def test_compensated_sum_matches_the_kahan_model_and_keeps_small_updates(ng, dtype):
    rng = np.random.default_rng(17)
    shape = (96, 200)
    s = rng.normal(0, 1, shape).astype(dtype)
    c = np.zeros(shape, dtype)
    dS, dC = ng.array(s, dtype=dtype), ng.array(c, dtype=dtype)
    naive = s.copy()
    exact = s.astype(np.float64)
    for i in range(40):
        a = (rng.normal(0, 1, shape) * 2.0 ** -9).astype(dtype)      # far below one ulp of most sums (fp16)
        ng.compensated_sum(dS, dC, ng.array(a, dtype=dtype), cmp_scale=1.0, add_scale=0.5)
        s, c = _kahan_model(s, c, a, 1.0, 0.5)
        naive = (naive.astype(np.float32) + a.astype(np.float32) * np.float32(0.5)).astype(dtype)
        exact += a.astype(np.float64) * 0.5
        assert np.array_equal(dS.get(), s), "sum after %d steps" % (i + 1)
        assert np.array_equal(dC.get(), c), "compensation after %d steps" % (i + 1)
    assert dC.kahan_count == 40
    if dtype is np.float16:
        # the point of the compensation: the fp16 running sum stays close to the exact one
        err_kahan = np.abs(s.astype(np.float64) - exact).mean()
        err_naive = np.abs(naive.astype(np.float64) - exact).mean()
        assert err_kahan < 0.25 * err_naive
    # kahan_reset: after that many steps the old compensation is dropped (cmp_scale = 0)
    dC.kahan_reset = 2
    dC.kahan_count = 3
    a = (rng.normal(0, 1, shape) * 2.0 ** -9).astype(dtype)
    ng.compensated_sum(dS, dC, ng.array(a, dtype=dtype))
    s2, c2 = _kahan_model(s, c, a, 0.0, 1.0)
    assert np.array_equal(dS.get(), s2) and np.array_equal(dC.get(), c2) and dC.kahan_count == 1
