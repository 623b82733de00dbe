"""Error paths that need a device: a bounded wait that runs out, scratch memory that grows under a
recorded sequence (B200 only). Nothing here faults or hangs the GPU: the wait gives up by itself."""
import ctypes

import numpy as np
import pytest

from nervanagpu_b200 import NervanaGPU, _lib
from oracle import reference_math as rm
from tests._util import rn16_tol

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_is_reported_and_the_context_stays_usable(ng, lib):
    ng.synchronize()
    waited = ng.zeros((2,), dtype=np.uint32)          # one 64-bit counter
    limit_ns = 2 * 1000 * 1000                          # 2 ms
    _lib.check(lib.ng_test_wait_expires(limit_ns, waited.ptr, None))
    rc = lib.ng_sync()
    assert rc == -6, "expected NG_ERR_TIMEOUT, got %d" % rc
    assert b"site 105" in lib.ng_last_error()
    w = waited.get()
    waited_ns = int(w[0]) | (int(w[1]) << 32)
    assert limit_ns <= waited_ns < 1000 * 1000 * 1000   # gave up after the limit, long before a second
    # the status word was cleared by the report, and ordinary work runs as before
    assert lib.ng_sync() == 0
    code = ctypes.c_int(-1)
    assert lib.ng_device_status(ctypes.byref(code)) == 0 and code.value == 0
    rng = np.random.default_rng(1)
    A = rng.normal(0, 1, (128, 256)).astype(np.float16)
    B = rng.normal(0, 1, (256, 192)).astype(np.float16)
    C = ng.empty((128, 192))
    ng.dot(ng.array(A), ng.array(B), C)
    ref = rm.gemm(A, B)
    assert (np.abs(C.get().astype(np.float32) - ref) <= rn16_tol(ref, rm.gemm_abs(A, B), 256)).all()
    assert lib.ng_sync() == 0
    # a limit can be set and reset for the library's own kernels
    _lib.check(lib.ng_set_wait_limit_ns(500 * 1000 * 1000))
    ng.dot(ng.array(A), ng.array(B), C)
    assert lib.ng_sync() == 0
    _lib.check(lib.ng_set_wait_limit_ns(0))


def test_replay_survives_growth_of_the_scratch_memory():
    """A recorded split-K GEMM keeps the scratch pointer it was recorded with. A later, larger
    call on the same stream makes the scratch grow; the recording must still give the right result."""
    ng = NervanaGPU(stochastic_round=False)
    ng.stream = ng.new_stream()
    rng = np.random.default_rng(11)
    hA = rng.normal(0, 0.1, (128, 8192)).astype(np.float16)
    hB = rng.normal(0, 0.1, (8192, 128)).astype(np.float16)
    A, B, C = ng.array(hA), ng.array(hB), ng.empty((128, 128))

    def small():
        ng.dot(A, B, C)                                # one tile, long k: split-K partials in scratch

    small()
    want = C.get()
    seq = ng.capture(small)
    # a much larger split-K problem on the same stream: its partials need more scratch
    bigA = ng.array(rng.normal(0, 0.1, (1024, 16384)).astype(np.float16))
    bigB = ng.array(rng.normal(0, 0.1, (16384, 512)).astype(np.float16))
    bigC = ng.empty((1024, 512))
    ng.dot(bigA, bigB, bigC)
    filler = [ng.zeros((1 << 20,), dtype=np.float32) for _ in range(8)]   # would reuse freed memory
    C.fill(0.0)
    seq.launch()
    ng.synchronize()
    assert np.array_equal(C.get(), want)
    ref = rm.gemm(hA, hB)
    assert (np.abs(want.astype(np.float32) - ref) <= rn16_tol(ref, rm.gemm_abs(hA, hB), 8192)).all()
    seq.release()
    del filler
