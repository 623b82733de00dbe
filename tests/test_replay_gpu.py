"""Recorded sequences (NervanaGPU.capture): a replay must give what the live calls give (B200 only)."""
import numpy as np
import pytest

from nervanagpu_b200 import NervanaGPU, _lib
from nervanagpu_b200.convnet import ConvStack

pytestmark = pytest.mark.gpu

TINY = {"name": "tiny_stack", "N": 64, "C": 3, "H": 19, "W": 19,
        "layers": [("conv", (64, 3, 3, 1, 1)), ("pool", (3, 3, 2)), ("conv", (32, 3, 3, 1, 1))]}


@pytest.fixture()
def streamed():
    ng = NervanaGPU(stochastic_round=False)
    ng.stream = ng.new_stream()
    return ng


def test_replay_matches_live_calls(streamed):
    ng = streamed
    rng = np.random.default_rng(5)
    a = ng.array(rng.normal(0, 1, (96, 64)).astype(np.float16))
    b = ng.array(rng.normal(0, 1, (64, 128)).astype(np.float16))
    c = ng.empty((96, 128))
    d = ng.empty((96, 128))

    def work():
        ng.dot(a, b, c, relu=True)
        d[:] = c * 0.5 + 1

    work()                                   # sizes scratch memory, compiles the element-wise kernel
    live = d.get()
    seq = ng.capture(work)
    a.set(rng.normal(0, 1, (96, 64)).astype(np.float16))      # new contents, same buffers
    seq.launch()
    replayed = d.get()
    work()
    assert np.array_equal(replayed, d.get())
    assert not np.array_equal(replayed, live)
    seq.release()


def test_capture_needs_a_stream_and_counts_launches(streamed):
    ng = streamed
    x = ng.ones((64, 64))

    def work():
        x[:] = x + 1

    work()
    lib = ng.lib

    def count():
        import ctypes
        n = ctypes.c_ulonglong()
        _lib.check(lib.ng_launch_count(ctypes.byref(n)))
        return n.value

    n0 = count()
    seq = ng.capture(work)
    assert count() == n0                     # recording runs nothing
    seq.launch()
    seq.launch()
    assert count() == n0 + 2
    assert float(x.get()[0, 0]) == 4.0       # 1 + live call + two replays
    plain = NervanaGPU(stochastic_round=False)
    with pytest.raises(_lib.NervanaError):
        plain.capture(lambda: None)          # default stream


def test_relu_mask_fused_into_pool_backward_changes_nothing():
    def run(fuse):
        ng = NervanaGPU(stochastic_round=False)
        stack = ConvStack(ng, TINY, seed=11)
        stack.fuse_relu_mask = fuse
        for _ in range(2):
            stack.step()
        return stack.weights_flat.get(), stack.grads_flat.get()

    w0, g0 = run(False)
    w1, g1 = run(True)
    assert np.array_equal(g0, g1)
    assert np.array_equal(w0, w1)


def test_weight_updates_on_a_side_stream_change_nothing():
    def run(overlap):
        ng = NervanaGPU(stochastic_round=False)
        ng.stream = ng.new_stream()
        stack = ConvStack(ng, TINY, seed=11)
        assert stack.overlap_update
        stack.overlap_update = overlap
        for _ in range(3):
            stack.step()
        return stack.weights_flat.get(), stack.grads_flat.get()

    w0, g0 = run(False)
    w1, g1 = run(True)
    assert np.array_equal(g0, g1)
    assert np.array_equal(w0, w1)


def test_recorded_training_step_equals_live_step():
    def run(record):
        ng = NervanaGPU(stochastic_round=False)
        ng.stream = ng.new_stream()
        stack = ConvStack(ng, TINY, seed=11)
        stack.step()
        if record:
            stack.record_steps()
        for _ in range(3):
            stack.step_prefetched()
        return stack.weights_flat.get(), stack.acts[-1].get()

    w_live, act_live = run(False)
    w_rec, act_rec = run(True)
    assert np.array_equal(w_live, w_rec)
    assert np.array_equal(act_live, act_rec)


def test_network_driver_runs_a_small_network_through_the_layer_classes():
    from nervanagpu_b200 import convnet_benchmarks as cb
    cb.NETWORKS["tiny"] = (1, [cb._data(64, 3, 20), cb._conv(32, 3, pad=1), cb._pool(2, 2), cb._conv(64, 3, pad=1),
                               cb._pool(2, 2), cb._full(96), cb._full(40)])
    lines = []
    try:
        res = cb.run_network(NervanaGPU(stochastic_round=False), "tiny", loops=2, out=lines.append)
    finally:
        del cb.NETWORKS["tiny"]
    assert set(res) == {"fprop", "bprop", "total"}
    assert all(ms > 0 and gflops > 0 for ms, gflops in res.values())
    assert sum(l.startswith("Avg(2)") for l in lines) == 3
