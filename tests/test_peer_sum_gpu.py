"""Gradient sum over peer memory fused with the SGD step (ng_peer_*): a group of one GPU here;
groups of 2 and 4 GPUs are checked by every multi-GPU bench run against a host-side sum."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_group_of_one_sums_its_own_gradient_and_steps_the_weights(ng, lib):
    group = ctypes.c_void_p()
    handle = ctypes.create_string_buffer(lib.ng_peer_handle_bytes())
    assert lib.ng_peer_create(ctypes.byref(group), 1, 0, handle) == 0
    try:
        assert lib.ng_peer_connect(group, handle.raw) == 0
        rng = np.random.default_rng(77)
        for n in (23232, 307200, 8, 1000, 4 * 3 + 2):      # whole vectors, and a ragged tail
            g = rng.normal(0, 1, n).astype(np.float32)
            w = rng.normal(0, 0.1, n).astype(np.float16)
            dg, dw = ng.array(g, dtype=np.float32), ng.array(w)
            lr = np.float32(-0.01)
            for launch in range(3):                           # both staging halves, and their reuse
                assert lib.ng_peer_sum_sgd_f32(group, dg.ptr, dw.ptr, n, float(lr), ng.stream) == 0
                w = (w.astype(np.float32) + g * lr).astype(np.float16)
            assert lib.ng_sync() == 0
            np.testing.assert_array_equal(dg.get(), g)
            np.testing.assert_array_equal(dw.get(), w)
            # no weights: the sum only
            assert lib.ng_peer_sum_sgd_f32(group, dg.ptr, None, n, 0.0, ng.stream) == 0
            assert lib.ng_sync() == 0
            np.testing.assert_array_equal(dg.get(), g)
        too_many = lib.ng_peer_max_bytes() // 4 + 4
        assert lib.ng_peer_sum_sgd_f32(group, dg.ptr, None, too_many, 0.0, ng.stream) != 0
    finally:
        assert lib.ng_peer_destroy(group) == 0
