"""ng_hgemm_static_scratch: the GEMM entry point for callers that cannot allocate device memory
(their memory is owned by a pool of their own, or cudaMalloc is off limits where they call us).

It keeps its split-K partial sums in a fixed array inside the library instead of a cudaMalloc'ed
workspace. The tests call it through the C ABI twice in a row and compare each result with
ng_hgemm on the same operands, within the tolerance the GEMM tests use (the two entry points
may split the reduction differently, so fp32 summation order can differ), and check that the
device's free memory does not move across a call. This file sorts last so that a run that stops
at the first failure has already run every other test.
"""
import ctypes

import numpy as np
import pytest

from oracle import reference_math as rm
from tests._util import rn16_tol

pytestmark = pytest.mark.gpu


def _call(fn, A, B, C, a_t, b_t, m, n, k, alpha=1.0, beta=0.0, relu=0, sr_bits=0, seed=0, offset=0):
    lda = A.shape[1]
    ldb = B.shape[1]
    return fn(A.ptr, B.ptr, C.ptr, a_t, b_t, m, n, k, lda, ldb, n, alpha, beta, relu, sr_bits, seed, offset, None)


def _free_bytes(lib):
    free, total = ctypes.c_size_t(), ctypes.c_size_t()
    assert lib.ng_mem_info(ctypes.byref(free), ctypes.byref(total)) == 0
    return free.value


@pytest.mark.parametrize("op,m,n,k", [("nn", 256, 128, 4096), ("tn", 384, 512, 2048), ("nt", 1000, 128, 1024),
                                      ("nn", 192, 48, 64), ("tn", 128, 64, 40)])
def test_matches_ng_hgemm_on_two_calls_in_a_row(ng, lib, op, m, n, k):
    """Includes k <= 64 (a single block of k: no partial sums, stored directly) and n <= 64."""
    rng = np.random.default_rng(2024)
    a_t, b_t = int(op[0] == "t"), int(op[1] == "t")
    hA = rng.normal(0, 0.1, (k, m) if a_t else (m, k)).astype(np.float16)
    hB = rng.normal(0, 0.1, (n, k) if b_t else (k, n)).astype(np.float16)
    hA2 = rng.normal(0, 0.1, hA.shape).astype(np.float16)
    A, B, A2 = ng.array(hA), ng.array(hB), ng.array(hA2)
    ref_c, new_c = ng.empty((m, n)), ng.empty((m, n))
    # second call uses other data, so stale partial sums from the first would show
    for i, (dA, host_a) in enumerate(((A, hA), (A2, hA2))):
        new_c.fill(-1.0)
        assert _call(lib.ng_hgemm, dA, B, ref_c, a_t, b_t, m, n, k, relu=1) == 0
        ng.synchronize()
        before = _free_bytes(lib)
        rc = _call(lib.ng_hgemm_static_scratch, dA, B, new_c, a_t, b_t, m, n, k, relu=1)
        assert rc == 0, lib.ng_last_error().decode()
        ng.synchronize()
        if i > 0:      # (the first call on a device may load the module's static data)
            assert _free_bytes(lib) == before, "the call changed the device's free memory"
        want, got = ref_c.get().astype(np.float32), new_c.get().astype(np.float32)
        tol = rn16_tol(want, rm.gemm_abs(host_a, hB, bool(a_t), bool(b_t)), k)
        assert (np.abs(got - want) <= tol).all()
        oracle = rm.gemm(host_a, hB, bool(a_t), bool(b_t), relu=True)
        assert (np.abs(got - oracle) <= tol).all()
    code = ctypes.c_int(-1)
    assert lib.ng_static_scratch_status(ctypes.byref(code)) == 0 and code.value == 0


def test_beta_term_and_stochastic_rounding(ng, lib):
    m, n, k = 256, 256, 1024
    rng = np.random.default_rng(7)
    hA = rng.normal(0, 0.1, (m, k)).astype(np.float16)
    hB = rng.normal(0, 0.1, (k, n)).astype(np.float16)
    hC = rng.normal(0, 1, (m, n)).astype(np.float16)
    A, B = ng.array(hA), ng.array(hB)
    ref_c, new_c = ng.array(hC), ng.array(hC)
    assert _call(lib.ng_hgemm, A, B, ref_c, 0, 0, m, n, k, alpha=0.5, beta=0.25) == 0
    assert _call(lib.ng_hgemm_static_scratch, A, B, new_c, 0, 0, m, n, k, alpha=0.5, beta=0.25) == 0
    ng.synchronize()
    oracle = rm.gemm(hA, hB, alpha=0.5, beta=0.25, C=hC)
    tol = rn16_tol(oracle, 0.5 * rm.gemm_abs(hA, hB) + 0.25 * np.abs(hC.astype(np.float32)), k)
    assert (np.abs(new_c.get().astype(np.float32) - oracle) <= tol).all()
    assert (np.abs(new_c.get().astype(np.float32) - ref_c.get().astype(np.float32)) <= tol).all()
    # stochastic rounding: every result is one of the two fp16 neighbours of the fp32 value
    sr_c = ng.empty((m, n))
    assert _call(lib.ng_hgemm_static_scratch, A, B, sr_c, 0, 0, m, n, k, sr_bits=10, seed=0xB200, offset=3) == 0
    ng.synchronize()
    exact = rm.gemm(hA, hB)
    got = sr_c.get().astype(np.float32)
    eps = k * 2.0 ** -24 * rm.gemm_abs(hA, hB)        # the fp32 sums themselves differ by summation order
    lo_a, _ = rm.fp16_neighbours(exact - np.sign(exact) * eps)
    _, hi_b = rm.fp16_neighbours(exact + np.sign(exact) * eps)
    lo = np.minimum(lo_a.astype(np.float32), hi_b.astype(np.float32))
    hi = np.maximum(lo_a.astype(np.float32), hi_b.astype(np.float32))
    assert ((got >= lo) & (got <= hi)).all()
    assert (got != exact.astype(np.float16)).any()    # it did round stochastically somewhere


def test_rejects_what_does_not_fit(ng, lib):
    m = n = 2048                     # 2 * m * n * 4 bytes = 32 MiB > the 16 MiB array
    A, B, C = ng.empty((m, 64)), ng.empty((64, n)), ng.empty((m, n))
    rc = _call(lib.ng_hgemm_static_scratch, A, B, C, 0, 0, m, n, 64)
    assert rc == -8 and b"static scratch" in lib.ng_last_error()
    # unaligned leading dimension: refused, not silently re-routed
    A2, B2, C2 = ng.empty((16, 20)), ng.empty((20, 12)), ng.empty((16, 12))
    assert _call(lib.ng_hgemm_static_scratch, A2, B2, C2, 0, 0, 16, 12, 20) == -2
