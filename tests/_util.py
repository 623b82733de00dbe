"""Shared helpers of the parity tests: tolerances and golden-fixture loading."""
import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# Tolerance of a round-to-nearest fp16 result against the fp32 oracle value `ref`, for a dot
# product of length k whose terms have absolute sum `absdot`:
#   one fp16 rounding (2^-11 relative, taken as 2^-10) + fp32 accumulation in any order
#   (k * 2^-24 * sum|a||b|, the classic gamma_k bound) + fp16 subnormal spacing.
def rn16_tol(ref, absdot, k):
    return 2.0 ** -10 * np.abs(ref) + k * 2.0 ** -24 * absdot + 2.0 ** -24


def f32_tol(absdot, k):
    """fp32 output (weight gradients): accumulation-order error only."""
    return k * 2.0 ** -23 * absdot + 1e-30


def assert_close(got, ref, tol, what=""):
    got = np.asarray(got, dtype=np.float32)
    err = np.abs(got - ref)
    bad = err > tol
    if bad.any():
        i = np.unravel_index(np.argmax(err - tol), err.shape)
        raise AssertionError("%s: %d of %d outside tolerance; worst at %s: got %r ref %r tol %r" %
                             (what, int(bad.sum()), bad.size, i, got[i], ref[i], np.broadcast_to(tol, err.shape)[i]))


def ref_percent_error(got, ref):
    """The reference's own figure of merit: 100 * max|diff| / mean|ref| (benchmarks/cublas_test.py:169-173)."""
    return 100.0 * np.abs(np.asarray(got, np.float32) - ref).max() / np.abs(ref).mean()


def golden(name):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


def golden_names(prefix):
    return sorted(f[:-4] for f in os.listdir(GOLDEN) if f.startswith(prefix) and f.endswith(".npz"))
