"""Conv + pool stacks of the benchmark networks and the loop that times them.

Follows the reference's benchmark driver (benchmarks/convnet-benchmarks.py:250-403) for the
convolutional part of its networks: forward chain with the ReLU fused into each convolution,
backward chain in reverse with, per convolution, the ReLU mask on the incoming deltas
(Layer.bprop_relu), bprop_conv (skipped for the first layer, which needs no input gradient),
update_conv, and the SGD step (nervanagpu/layers.py:87-96,483-502). Weights and weight gradients
of all layers live in two flat buffers so that one all-reduce and one fused SGD kernel serve the
whole stack when the minibatch is split over several GPUs.
"""
import ctypes

import numpy as np

from . import _lib
from .layers import ConvLayer

# (kind, params): conv = (K, R, S, pad, stride), pool = (R, S, stride)
ALEXNET = {
    "name": "alexnet_conv_stack", "N": 128, "C": 3, "H": 224, "W": 224,
    "layers": [("conv", (64, 11, 11, 2, 4)), ("pool", (3, 3, 2)),
               ("conv", (192, 5, 5, 2, 1)), ("pool", (3, 3, 2)),
               ("conv", (384, 3, 3, 1, 1)), ("conv", (256, 3, 3, 1, 1)), ("conv", (256, 3, 3, 1, 1)),
               ("pool", (3, 3, 2))],
}
VGG_A = {
    "name": "vgg_a_conv_stack", "N": 64, "C": 3, "H": 224, "W": 224,
    "layers": [("conv", (64, 3, 3, 1, 1)), ("pool", (2, 2, 2)),
               ("conv", (128, 3, 3, 1, 1)), ("pool", (2, 2, 2)),
               ("conv", (256, 3, 3, 1, 1)), ("conv", (256, 3, 3, 1, 1)), ("pool", (2, 2, 2)),
               ("conv", (512, 3, 3, 1, 1)), ("conv", (512, 3, 3, 1, 1)), ("pool", (2, 2, 2)),
               ("conv", (512, 3, 3, 1, 1)), ("conv", (512, 3, 3, 1, 1)), ("pool", (2, 2, 2))],
}
NETWORKS = {"alexnet": ALEXNET, "vgg_a": VGG_A}


def shard_minibatch(array, rank, world):
    """The slice of a (..., N) host array that rank `rank` of `world` works on: images are the
    innermost dimension of every activation, so a shard is a contiguous copy of N/world columns.
    N/world must stay a multiple of 8 (the convolution kernels' requirement)."""
    n = array.shape[-1]
    if n % world != 0 or (n // world) % 8 != 0:
        raise ValueError("minibatch of %d cannot be split over %d ranks in multiples of 8" % (n, world))
    per = n // world
    return np.ascontiguousarray(array[..., rank * per:(rank + 1) * per])


def bucket_layout(sizes, align=8):
    """Offsets of per-layer slices inside one flat buffer (elements). Every slice starts on an
    `align`-element boundary so that each view stays 16-byte aligned for fp16 and fp32 alike."""
    offsets, total = [], 0
    for s in sizes:
        offsets.append(total)
        total += (s + align - 1) // align * align
    return offsets, total


def comm_bucket_order(sizes, small_fraction=0.15):
    """Gradient buckets of the multi-GPU step as (first layer, one past the last layer), in the
    order in which the backward pass completes them: the upper layers, which hold most of the
    parameters (everything above the lowest layers that together hold at most `small_fraction`), form one
    bucket; the layers below it go one by one, so that what is exposed at the end of the step is
    the sum of the first layer's few weights only."""
    n = len(sizes)
    if n <= 1:
        return [(0, n)] if n else []
    split = 1
    while split + 1 < n and sum(sizes[:split + 1]) <= small_fraction * sum(sizes):
        split += 1
    return [(split, n)] + [(i, i + 1) for i in range(split - 1, -1, -1)]


class ConvStack(object):
    """A chain of ConvLayer / PoolLayer objects with their activations, deltas and weights."""

    def __init__(self, ng, net, N=None, seed=1003, learning_rate=-1e-4, comm=None, shard=None, data_seed=None):
        """`shard=(rank, world)`: the minibatch of net["N"] images is generated whole (same seed on
        every rank) and this rank keeps its slice of N/world images (a minibatch split over GPUs).
        Weights always come from `seed`, so ranks that share it start from identical weights; the
        data of an unsharded stack comes from `data_seed` (default: `seed`)."""
        self.ng = ng
        self.net = net
        self.shard = shard
        if shard is not None:
            N = net["N"] // shard[1]
        self.N = N = net["N"] if N is None else N
        self.comm = comm                      # ng_comm handle or None (single GPU)
        # ng_peer group (gradient sums over peer memory, fused with the SGD step) or None: used for
        # the small, late buckets, whose cost is latency; the big first bucket stays with NCCL
        self.peer = None
        self.peer_max_bytes = 0
        self.lr = learning_rate
        rng = np.random.default_rng(seed)
        C, H, W = net["C"], net["H"], net["W"]
        self.layers = []
        for kind, prm in net["layers"]:
            if kind == "conv":
                K, R, S, pad, stride = prm
                layer = ng.conv_layer(np.float16, N, C, K, 1, H, W, 1, R, S, 0, pad, pad, 1, stride, stride)
                C, H, W = K, layer.P, layer.Q
            else:
                R, S, stride = prm
                layer = ng.pool_layer(np.float16, "max", N, C, 1, H, W, 1, 1, R, S, 0, 0, 0, 0, 1, 1, stride, stride)
                H, W = layer.P, layer.Q
            self.layers.append(layer)
        self.convs = [l for l in self.layers if isinstance(l, ConvLayer)]

        # flat weight / gradient buffers with per-layer views
        offsets, total_f = bucket_layout([l.sizeF for l in self.convs])
        self.weights_flat = ng.empty((total_f,), dtype=np.float16)
        self.grads_flat = ng.zeros((total_f,), dtype=np.float32)
        w_host = np.zeros(total_f, dtype=np.float16)
        for l, off in zip(self.convs, offsets):
            w_host[off:off + l.sizeF] = rng.normal(0.0, 0.01, l.sizeF).astype(np.float16)
            l.weights = self.weights_flat[off:off + l.sizeF].reshape(l.dimF)
            l.updat_out = self.grads_flat[off:off + l.sizeF].reshape(l.dimF)
        self.weights_flat.set(w_host)

        # activations and deltas
        self.input = ng.empty(self.layers[0].dimI, dtype=np.float16)
        self.acts = [ng.empty(l.dimO, dtype=np.float16) for l in self.layers]
        self.deltas = [None] + [ng.empty(l.dimI, dtype=np.float16) for l in self.layers[1:]]
        self.top_delta = ng.empty(self.layers[-1].dimO, dtype=np.float16)
        drng = rng if data_seed is None else np.random.default_rng(data_seed)
        if shard is None:
            self.host_input = drng.uniform(0.0, 1.0, self.layers[0].dimI).astype(np.float16)
            top = (drng.uniform(-1.0, 1.0, self.layers[-1].dimO) * 0.125).astype(np.float16)
        else:
            rank, world = shard
            whole_in = self.layers[0].dimI[:-1] + (net["N"],)
            whole_top = self.layers[-1].dimO[:-1] + (net["N"],)
            self.host_input = shard_minibatch(drng.uniform(0.0, 1.0, whole_in).astype(np.float16), rank, world)
            top = shard_minibatch((drng.uniform(-1.0, 1.0, whole_top) * 0.125).astype(np.float16), rank, world)
        self.input.set(self.host_input)
        self.top_delta.set(top)
        # pooling layers keep their windows' argmax between the forward and the backward pass
        self.argmax = [None] * len(self.layers)
        for i, l in enumerate(self.layers):
            if not isinstance(l, ConvLayer):
                nbytes = ng.pool_argmax_bytes(l)
                if nbytes:
                    self.argmax[i] = ng.empty((nbytes,), dtype=np.uint8)
        self.probe = None    # optional callable(name, layer, launch) used to time single launches
        self.fuse_relu_mask = True   # False: every ReLU mask is its own element-wise kernel, as in the reference
        # weight updates on a second stream beside the backward chain (needs a stream of the
        # backend's own: work on the default stream would serialise with it anyway)
        self.overlap_update = ng.stream is not None
        self._side, self._side_busy = None, False
        self._comm_stream, self._comm_busy = None, False
        # Gradient buckets of the multi-GPU step, as ranges of the flat buffers: the upper layers
        # (most of the parameters) are summed over the GPUs as soon as the lowest of them has its
        # gradient, while the layers below still compute; the small remainder follows. Each
        # bucket's SGD step runs on the communication stream right behind its sum.
        self._conv_offsets = offsets
        self._flat_elems = total_f
        self.comm_buckets = comm_bucket_order([l.sizeF for l in self.convs])

        # work per step on this GPU: fprop + update for every conv, bprop for all but the first
        self.flops_fprop = sum(l.flops for l in self.convs)
        self.flops_bprop = sum(l.flops for l in self.convs[1:]) + sum(l.flops for l in self.convs)
        self.flops = self.flops_fprop + self.flops_bprop

    # ------------------------------------------------------------------------------------
    def _run(self, name, layer, launch):
        if self.probe is not None:
            self.probe(name, layer, launch)
        else:
            launch()

    def fprop(self):
        ng = self.ng
        x = self.input
        for i, l in enumerate(self.layers):
            y = self.acts[i]
            if isinstance(l, ConvLayer):
                self._run("fprop_conv", l, lambda l=l, x=x, y=y: ng.fprop_conv(l, x, l.weights, y, relu=True))
            else:
                self._run("fprop_pool", l, lambda l=l, x=x, y=y, a=self.argmax[i]: ng.fprop_pool(l, x, y, argmax=a))
            x = y
        return x

    def bprop(self):
        ng = self.ng
        grad = self.top_delta
        masked = False     # grad already carries the ReLU mask of the conv layer it belongs to
        for i in range(len(self.layers) - 1, -1, -1):
            l = self.layers[i]
            x = self.input if i == 0 else self.acts[i - 1]
            dx = self.deltas[i]
            if isinstance(l, ConvLayer):
                y = self.acts[i]
                if not masked:
                    self._run("bprop_relu", l, lambda grad=grad, y=y: _relu_mask(grad, y))
                masked = False
                # The weight gradient is needed only at the end of the step, the input gradient by
                # the next layer down: with a side stream the update runs beside the backward chain
                # and fills the SMs that kernels with fewer than 148 tiles leave idle.
                side = self._fork_side() if self.overlap_update and self.probe is None else None
                if dx is not None:
                    self._run("bprop_conv", l, lambda l=l, grad=grad, dx=dx: ng.bprop_conv(l, l.weights, grad, dx))
                if side is not None:
                    main, ng.stream = ng.stream, side
                    try:
                        ng.update_conv(l, x, grad, l.updat_out)
                    finally:
                        ng.stream = main
                    ci = self.convs.index(l)
                    bucket = [b for b in self.comm_buckets if b[0] == ci]
                    if self.comm is not None and bucket:
                        # This layer is the lowest of its bucket: the bucket's gradients are summed
                        # over the GPUs and applied while the layers below are still computing (a
                        # third stream: the sum must not hold up the updates). The weights of the
                        # bucket are free once this layer's bprop_conv, queued above, has read them.
                        self._allreduce_behind(side, bucket[0])
                else:
                    self._run("update_conv", l, lambda l=l, x=x, grad=grad: ng.update_conv(l, x, grad, l.updat_out))
            else:
                # the pool reads the (ReLU) output of the conv below it anyway: its backward pass
                # applies that layer's mask as it writes the deltas
                fuse = self.fuse_relu_mask and i > 0 and isinstance(self.layers[i - 1], ConvLayer)
                self._run("bprop_pool", l, lambda l=l, x=x, grad=grad, dx=dx, fuse=fuse, a=self.argmax[i]:
                          ng.bprop_pool(l, x, grad, dx, relu_mask=fuse, argmax=a))
                masked = fuse
            grad = dx
        summed = self._comm_busy          # the buckets were summed and applied behind the updates
        self._join_side()
        if summed:
            return
        if self.comm is not None:
            self._run("allreduce_dW", None, self.allreduce_grads)
        self._run("grad_descent", None, self.grad_descent)

    def _bucket_range(self, bucket):
        first, last = bucket
        start = self._conv_offsets[first]
        end = self._conv_offsets[last] if last < len(self.convs) else self._flat_elems
        return start, end

    def _allreduce_behind(self, after_stream, bucket):
        ng, lib = self.ng, self.ng.lib
        if self._comm_stream is None:
            self._comm_stream = ng.new_stream()
            self._comm_ev, self._comm_done, self._w_free = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p()
            for ev in (self._comm_ev, self._comm_done, self._w_free):
                _lib.check(lib.ng_event_create(ctypes.byref(ev)))
        start, end = self._bucket_range(bucket)
        g, w = self.grads_flat[start:end], self.weights_flat[start:end]
        _lib.check(lib.ng_event_record(self._comm_ev, after_stream))      # the bucket's last update
        _lib.check(lib.ng_event_record(self._w_free, ng.stream))          # its last reader of the weights
        _lib.check(lib.ng_stream_wait_event(self._comm_stream, self._comm_ev))
        if self.peer is not None and g.nbytes <= self.peer_max_bytes:
            # one kernel per GPU: copy to the staging buffer the peers have mapped, sum their copies
            # in rank order, apply the step (the weights must be free first)
            _lib.check(lib.ng_stream_wait_event(self._comm_stream, self._w_free))
            _lib.check(lib.ng_peer_sum_sgd_f32(self.peer, g.ptr, w.ptr, g.size, self.lr, self._comm_stream))
            self._comm_busy = True
            return
        _lib.check(lib.ng_comm_allreduce_f32(self.comm, g.ptr, g.size, self._comm_stream))
        _lib.check(lib.ng_stream_wait_event(self._comm_stream, self._w_free))
        main, ng.stream = ng.stream, self._comm_stream
        try:
            w[:] = w + g * self.lr
        finally:
            ng.stream = main
        self._comm_busy = True

    def _fork_side(self):
        """The side stream, made to wait for everything queued on the main stream so far."""
        lib = self.ng.lib
        if self._side is None:
            self._side = self.ng.new_stream()
            self._fork_ev, self._join_ev = ctypes.c_void_p(), ctypes.c_void_p()
            _lib.check(lib.ng_event_create(ctypes.byref(self._fork_ev)))
            _lib.check(lib.ng_event_create(ctypes.byref(self._join_ev)))
        _lib.check(lib.ng_event_record(self._fork_ev, self.ng.stream))
        _lib.check(lib.ng_stream_wait_event(self._side, self._fork_ev))
        self._side_busy = True
        return self._side

    def _join_side(self):
        if self._side_busy:
            lib = self.ng.lib
            _lib.check(lib.ng_event_record(self._join_ev, self._side))
            _lib.check(lib.ng_stream_wait_event(self.ng.stream, self._join_ev))
            self._side_busy = False
        if self._comm_busy:
            lib = self.ng.lib
            _lib.check(lib.ng_event_record(self._comm_done, self._comm_stream))
            _lib.check(lib.ng_stream_wait_event(self.ng.stream, self._comm_done))
            self._comm_busy = False

    def allreduce_grads(self):
        _lib.check(self.ng.lib.ng_comm_allreduce_f32(self.comm, self.grads_flat.ptr, self.grads_flat.size,
                                                     self.ng.stream))

    def grad_descent(self):
        # one fused kernel over the flat buffers: weights += grads * learning_rate
        w, g = self.weights_flat, self.grads_flat
        w[:] = w + g * self.lr

    def step(self):
        self.fprop()
        self.bprop()

    def set_input(self, host_array):
        self.input.set(host_array)

    # ---- pipelined input: the next minibatch is copied while the current step computes -------
    def _init_prefetch(self):
        lib = self.ng.lib
        self._copy_stream = ctypes.c_void_p()
        _lib.check(lib.ng_stream_create(ctypes.byref(self._copy_stream)))
        self._next_input = self.ng.empty(self.layers[0].dimI, dtype=np.float16)
        self._copied, self._consumed = ctypes.c_void_p(), ctypes.c_void_p()
        _lib.check(lib.ng_event_create(ctypes.byref(self._copied)))
        _lib.check(lib.ng_event_create(ctypes.byref(self._consumed)))
        self._prefetch_pending = False
        self._consumed_recorded = False

    def record_steps(self):
        """Record one step per input buffer (the live one and the prefetch spare); step_prefetched
        then replays the recording that reads the buffer it swapped in. step() must have run before.
        With several GPUs the NCCL all-reduces are part of the recording (every rank must record
        and replay the same sequence)."""
        if not hasattr(self, "_copy_stream"):
            self._init_prefetch()
        probe, self.probe = self.probe, None
        live = self.input
        self._recorded = {}
        try:
            for buf in (live, self._next_input):
                self.input = buf
                self._recorded[buf.ptr] = self.ng.capture(self.step)
        finally:
            self.input = live
            self.probe = probe

    def prefetch_input(self, pinned_host_ptr):
        """Start the host-to-device copy of the next minibatch (pinned host memory) on a separate
        stream into the spare input buffer. It overlaps whatever the compute stream is doing."""
        if not hasattr(self, "_copy_stream"):
            self._init_prefetch()
        lib = self.ng.lib
        if self._consumed_recorded:
            # the spare buffer was the live input until the step that recorded this event finished
            _lib.check(lib.ng_stream_wait_event(self._copy_stream, self._consumed))
        _lib.check(lib.ng_memcpy_h2d_async(self._next_input.ptr, pinned_host_ptr, self._next_input.nbytes,
                                           self._copy_stream))
        _lib.check(lib.ng_event_record(self._copied, self._copy_stream))
        self._prefetch_pending = True

    def step_prefetched(self):
        """Swap in the prefetched minibatch (waiting for its copy on the device, not on the host)
        and run one step."""
        lib = self.ng.lib
        if getattr(self, "_prefetch_pending", False):
            _lib.check(lib.ng_stream_wait_event(self.ng.stream, self._copied))
            self.input, self._next_input = self._next_input, self.input
            self._prefetch_pending = False
            # everything queued so far (the previous step, which read what is now the spare
            # buffer) is done when this event fires; the next copy waits for it, not for this step
            _lib.check(lib.ng_event_record(self._consumed, self.ng.stream))
            self._consumed_recorded = True
        recorded = getattr(self, "_recorded", None)
        if recorded:
            recorded[self.input.ptr].launch()
        else:
            self.step()


def _relu_mask(grad, act):
    grad[:] = grad * (act > 0)


class StepTimer(object):
    """CUDA-event timing of a callable on the backend's stream."""

    def __init__(self, ng):
        self.ng = ng
        self.start, self.end = ctypes.c_void_p(), ctypes.c_void_p()
        _lib.check(ng.lib.ng_event_create(ctypes.byref(self.start)))
        _lib.check(ng.lib.ng_event_create(ctypes.byref(self.end)))

    def time_ms(self, fn, repeat):
        lib, stream = self.ng.lib, self.ng.stream
        _lib.check(lib.ng_event_record(self.start, stream))
        for _ in range(repeat):
            fn()
        _lib.check(lib.ng_event_record(self.end, stream))
        _lib.check(lib.ng_event_sync(self.end))
        ms = ctypes.c_float()
        _lib.check(lib.ng_event_elapsed_ms(self.start, self.end, ctypes.byref(ms)))
        return ms.value
