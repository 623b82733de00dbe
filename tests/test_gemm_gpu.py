"""ng.dot / the hgemm C entry points against the numpy oracle (B200 only)."""
import ctypes

import numpy as np
import pytest

from oracle import reference_math as rm
from tests._util import assert_close, ref_percent_error, rn16_tol

pytestmark = pytest.mark.gpu


def _operands(rng, m, n, k, op, std=1.0):
    A = rng.normal(0, std, (k, m) if op[0] == "t" else (m, k)).astype(np.float16)
    B = rng.normal(0, std, (n, k) if op[1] == "t" else (k, n)).astype(np.float16)
    return A, B


def _dot(ng, A, B, op, C0=None, **kw):
    dA, dB = ng.array(A), ng.array(B)
    m = A.shape[1] if op[0] == "t" else A.shape[0]
    n = B.shape[0] if op[1] == "t" else B.shape[1]
    dC = ng.array(C0) if C0 is not None else ng.empty((m, n))
    ng.dot(dA.T if op[0] == "t" else dA, dB.T if op[1] == "t" else dB, dC, **kw)
    return dC.get()


@pytest.mark.parametrize("size", [257, 256, 255, 129, 128, 127, 65, 64, 17, 16, 15])
@pytest.mark.parametrize("op", ["nn", "nt", "tn"])
def test_known_answers_all_ones_and_zeros(ng, size, op):
    """The reference's C smoke test (kernels/C_interface/test.cu:27-55,70): edge tiles, aligned and
    unaligned leading dimensions (the latter run on the SIMT kernel)."""
    ones = np.ones((size, size), dtype=np.float16)
    assert (_dot(ng, ones, ones, op) == size).all()
    zeros = np.zeros((size, size), dtype=np.float16)
    assert (_dot(ng, zeros, zeros, op) == 0).all()


def test_config1_tn_2048_relu(ng):
    """BASELINE config 1: C = relu(A^T B), A k x m, B k x n, m=n=k=2048, N(0,1), seed 1001."""
    rng = np.random.default_rng(1001)
    k = m = n = 2048
    A = rng.standard_normal((k, m)).astype(np.float16)
    B = rng.standard_normal((k, n)).astype(np.float16)
    got = _dot(ng, A, B, "tn", relu=True)
    ref = rm.gemm(A, B, a_t=True, relu=True)
    assert_close(got, ref, rn16_tol(ref, rm.gemm_abs(A, B, a_t=True), k), "cfg1")
    assert ref_percent_error(got, ref) <= 0.7   # the reference's fp16 threshold, cublas_test.py:96


@pytest.mark.parametrize("op", ["nn", "nt", "tn"])
@pytest.mark.parametrize("mnk", [(4096, 128, 9216), (4096, 128, 4096), (1000, 128, 4096), (9216, 4096, 128),
                                 (3072, 3072, 3072)])
def test_config2_fc_sweep(ng, op, mnk):
    """BASELINE config 2 shapes, inputs N(0, 0.1), round to nearest."""
    m, n, k = mnk
    if m * n * k > 2 ** 34:
        m, n, k = 1024, 1024, 3072      # full 3072^3 is covered by the linearity test below
    rng = np.random.default_rng(1002 + m + k)
    A, B = _operands(rng, m, n, k, op, std=0.1)
    got = _dot(ng, A, B, op)
    ref = rm.gemm(A, B, a_t=op[0] == "t", b_t=op[1] == "t")
    assert_close(got, ref, rn16_tol(ref, rm.gemm_abs(A, B, op[0] == "t", op[1] == "t"), k), "cfg2 %s %s" % (op, mnk))


@pytest.mark.parametrize("op", ["nn", "nt", "tn"])
def test_ragged_shapes_alpha_beta_relu(ng, op):
    """Odd sizes of the reference's gemm_test.py lists (:27-29), aligned to 8 where TMA needs it
    and not aligned otherwise; epilogue order alpha -> relu -> beta."""
    rng = np.random.default_rng(7)
    for (m, n, k) in [(136, 72, 200), (778, 192, 1536), (65, 127, 9), (1, 64, 192), (8, 8, 8), (785, 16, 72)]:
        A, B = _operands(rng, m, n, k, op)
        C0 = rng.standard_normal((m, n)).astype(np.float16)
        got = _dot(ng, A, B, op, C0=C0, alpha=0.5, beta=0.25, relu=True)
        ref = rm.gemm(A, B, op[0] == "t", op[1] == "t", alpha=0.5, beta=0.25, relu=True, C=C0)
        tol = rn16_tol(ref, rm.gemm_abs(A, B, op[0] == "t", op[1] == "t"), k) + 2.0 ** -11 * np.abs(C0.astype(np.float32))
        assert_close(got, ref, tol, "%s %s" % (op, (m, n, k)))


def test_simt_and_tensor_paths_agree(ng, lib):
    """Both kernels accumulate in fp32 and round once: results agree to one fp16 ulp."""
    rng = np.random.default_rng(3)
    m, n, k = 384, 256, 512
    A, B = _operands(rng, m, n, k, "nn")
    dA, dB = ng.array(A), ng.array(B)
    c1, c2 = ng.empty((m, n)), ng.empty((m, n))
    for fn, c in ((lib.ng_hgemm, c1), (lib.ng_hgemm_simt, c2)):
        assert fn(dA.ptr, dB.ptr, c.ptr, 0, 0, m, n, k, k, n, n, 1.0, 0.0, 0, 0, 0, 0, None) == 0
    a, b = c1.get().astype(np.float32), c2.get().astype(np.float32)
    # different summation orders: allow the fp32 accumulation slack on top of one fp16 ulp
    assert (np.abs(a - b) <= rn16_tol(a, rm.gemm_abs(A, B), k)).all()


def test_large_size_property_linearity(ng):
    """3072^3 at full size: dot(A, B1 + B2) == dot(A, B1) + dot(A, B2) within rounding, plus a
    sampled exact check of 64 rows against the oracle."""
    rng = np.random.default_rng(11)
    n = 3072
    A = rng.normal(0, 0.1, (n, n)).astype(np.float16)
    B1 = (rng.integers(-8, 9, (n, n)) / 16.0).astype(np.float16)
    B2 = (rng.integers(-8, 9, (n, n)) / 16.0).astype(np.float16)
    c1, c2, c12 = _dot(ng, A, B1, "nn"), _dot(ng, A, B2, "nn"), _dot(ng, A, (B1 + B2).astype(np.float16), "nn")
    s = c1.astype(np.float32) + c2.astype(np.float32)
    assert (np.abs(c12.astype(np.float32) - s) <= 3 * 2.0 ** -10 * (np.abs(s) + np.abs(c1) + np.abs(c2)) + 1e-3).all()
    rows = rng.choice(n, 64, replace=False)
    ref = rm.gemm(A[rows], B1)
    assert_close(c1[rows], ref, rn16_tol(ref, rm.gemm_abs(A[rows], B1), n), "sampled rows")


def test_batched_dot(ng):
    rng = np.random.default_rng(5)
    b, m, n, k = 4, 128, 256, 64
    A = rng.standard_normal((b, m, k)).astype(np.float16)
    B = rng.standard_normal((b, k, n)).astype(np.float16)
    dA, dB, dC = ng.array(A), ng.array(B), ng.empty((b, m, n))
    ng.batched_dot(dA, dB, dC)
    ref = np.einsum("bmk,bkn->bmn", A.astype(np.float32), B.astype(np.float32))
    assert_close(dC.get(), ref, 2.0 ** -10 * np.abs(ref) + 1e-2, "batched grid")
    # 2-D C: the products are summed over the batch
    dS = ng.empty((m, n))
    ng.batched_dot(dA, dB, dS)
    refs = ref.sum(axis=0)
    assert_close(dS.get(), refs, 2.0 ** -10 * np.abs(refs) + 2e-2, "batched loops")


def test_reference_c_interface(ng, lib):
    """nervana_hgemm / nervana_hgemm_colmajor keep the reference's signatures and conventions."""
    rng = np.random.default_rng(9)
    m, n, k = 128, 64, 256
    A, B = _operands(rng, m, n, k, "nn")
    dA, dB, dC = ng.array(A), ng.array(B), ng.empty((m, n))
    assert lib.nervana_loadKernels(b"unused")
    assert lib.nervana_randStateSizeBytes() == 2048 * 32 * 4
    assert lib.nervana_hgemm(dA.ptr, dB.ptr, dC.ptr, False, False, m, n, k, k, n, n, 1.0, 0.0, None, False, True, None, -1)
    ref = rm.gemm(A, B, relu=True)
    assert_close(dC.get(), ref, rn16_tol(ref, rm.gemm_abs(A, B), k), "nervana_hgemm")
    # column-major view of the same buffers: C^T (n x m col-major == m x n row-major) = B^T A^T
    dCt = ng.empty((m, n))
    assert lib.nervana_hgemm_colmajor(dB.ptr, dA.ptr, dCt.ptr, False, False, n, m, k, n, k, n, 1.0, 0.0, None,
                                      False, True, None, -1)
    assert np.array_equal(dCt.get(), dC.get())
    assert not lib.nervana_sgemm(dA.ptr, dB.ptr, dC.ptr, False, False, m, n, k, k, n, n, 1.0, 0.0, None, False, False,
                                 None, -1)


def test_dot_argument_errors(ng):
    A, B, C = ng.empty((16, 8)), ng.empty((8, 16)), ng.empty((16, 16))
    with pytest.raises(AssertionError):
        ng.dot(A.T, B.T, C)                      # "tt" is not supported
    with pytest.raises(AssertionError):
        ng.dot(A, ng.empty((9, 16)), C)          # inner dimensions differ
    with pytest.raises(TypeError):
        ng.dot(ng.empty((4, 4), dtype=np.float32), ng.empty((4, 4), dtype=np.float32),
               ng.empty((4, 4), dtype=np.float32))
    with pytest.raises(TypeError):
        ng.dot(ng.empty((4, 4), dtype=np.int8), ng.empty((4, 4), dtype=np.int8), ng.empty((4, 4), dtype=np.int8))


@pytest.mark.parametrize("op", ["nn", "nt", "tn"])
def test_cta_pair_instances_match_the_oracle(ng, lib, op):
    """The two-SM form of the tensor-core kernel (tcgen05 cta_group::2, switched on with the
    "pair_mma" tuning field): a 256-row tile is shared by the two CTAs of a cluster, each of which
    loads its own half of the B columns. Same results as the one-CTA kernel up to summation order."""
    rng = np.random.default_rng(31)
    try:
        assert lib.ng_tune(b"pair_mma", 1) == 0
        for (m, n, k) in [(512, 512, 256), (384, 256, 1024), (1000, 136, 520), (256, 128, 64)]:
            A, B = _operands(rng, m, n, k, op, std=0.1)
            C0 = rng.standard_normal((m, n)).astype(np.float16)
            got = _dot(ng, A, B, op, C0=C0, alpha=0.5, beta=0.25, relu=True)
            ref = rm.gemm(A, B, op[0] == "t", op[1] == "t", alpha=0.5, beta=0.25, relu=True, C=C0)
            tol = rn16_tol(ref, rm.gemm_abs(A, B, op[0] == "t", op[1] == "t"), k) + 2.0 ** -11 * np.abs(C0.astype(np.float32))
            assert_close(got, ref, tol, "pair %s %s" % (op, (m, n, k)))
            plain = _dot(ng, A, B, op)
            ref = rm.gemm(A, B, op[0] == "t", op[1] == "t")
            assert_close(plain, ref, rn16_tol(ref, rm.gemm_abs(A, B, op[0] == "t", op[1] == "t"), k), "pair plain")
    finally:
        assert lib.ng_tune(b"pair_mma", -1) == 0
    assert lib.ng_sync() == 0
