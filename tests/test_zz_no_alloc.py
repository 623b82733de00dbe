"""ng_hgemm_static_scratch: the GEMM entry point for callers that cannot allocate device memory
(their memory is owned by a pool of their own, or cudaMalloc is off limits where they call us).

It keeps its split-K partial sums in a fixed array inside the library instead of a cudaMalloc'ed
workspace. The test calls it through the C ABI twice in a row and compares each result with
ng_hgemm on the same operands, within the tolerance the GEMM tests use (the two entry points
may split the reduction differently, so fp32 summation order can differ). This file sorts last
so that a run that stops at the first failure has already run every other test.
"""
import ctypes

import numpy as np
import pytest

from oracle import reference_math as rm
from tests._util import rn16_tol

pytestmark = pytest.mark.gpu


def _call(fn, A, B, C, a_t, b_t, m, n, k, alpha=1.0, beta=0.0, relu=0):
    lda = A.shape[1]
    ldb = B.shape[1]
    return fn(A.ptr, B.ptr, C.ptr, a_t, b_t, m, n, k, lda, ldb, n, alpha, beta, relu, 0, 0, 0, None)


@pytest.mark.parametrize("op,m,n,k", [("nn", 256, 128, 4096), ("tn", 384, 512, 2048), ("nt", 1000, 128, 1024)])
def test_matches_ng_hgemm_on_two_calls_in_a_row(ng, lib, op, m, n, k):
    rng = np.random.default_rng(2024)
    a_t, b_t = int(op[0] == "t"), int(op[1] == "t")
    hA = rng.normal(0, 0.1, (k, m) if a_t else (m, k)).astype(np.float16)
    hB = rng.normal(0, 0.1, (n, k) if b_t else (k, n)).astype(np.float16)
    hA2 = rng.normal(0, 0.1, hA.shape).astype(np.float16)
    A, B, A2 = ng.array(hA), ng.array(hB), ng.array(hA2)
    ref_c, new_c = ng.empty((m, n)), ng.empty((m, n))
    # second call uses other data, so stale partial sums from the first would show
    for dA, host_a in ((A, hA), (A2, hA2)):
        new_c.fill(-1.0)
        assert _call(lib.ng_hgemm, dA, B, ref_c, a_t, b_t, m, n, k, relu=1) == 0
        rc = _call(lib.ng_hgemm_static_scratch, dA, B, new_c, a_t, b_t, m, n, k, relu=1)
        assert rc == 0, lib.ng_last_error().decode()
        ng.synchronize()
        want, got = ref_c.get().astype(np.float32), new_c.get().astype(np.float32)
        tol = rn16_tol(want, rm.gemm_abs(host_a, hB, bool(a_t), bool(b_t)), k)
        assert (np.abs(got - want) <= tol).all()
        oracle = rm.gemm(host_a, hB, bool(a_t), bool(b_t), relu=True)
        assert (np.abs(got - oracle) <= tol).all()


def test_rejects_what_does_not_fit(ng, lib):
    m = n = 2048                     # 2 * m * n * 4 bytes = 32 MiB > the 16 MiB array
    A, B, C = ng.empty((m, 64)), ng.empty((64, n)), ng.empty((m, n))
    rc = _call(lib.ng_hgemm_static_scratch, A, B, C, 0, 0, m, n, 64)
    assert rc == -8 and b"static scratch" in lib.ng_last_error()
    # unaligned leading dimension: refused, not silently re-routed
    A2, B2, C2 = ng.empty((16, 20)), ng.empty((20, 12)), ng.empty((16, 12))
    assert _call(lib.ng_hgemm_static_scratch, A2, B2, C2, 0, 0, 16, 12, 20) == -2
