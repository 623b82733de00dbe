"""Layer parameter objects and the thin network-layer helpers used by the benchmark harness.

ConvLayer / PoolLayer mirror the reference's parameter objects (nervanagpu/layers.py:279-506,
540-640): same constructor arguments, same derived attributes (M, P, Q, dimI/dimF/dimO, sizes,
flops, nOut) and the same assertions. What they no longer carry is the Maxwell launch detail
(grids, magic-number division constants, LUT sizes): they hold the C-ABI descriptor instead.
Layer / DataLayer / FullLayer chain fprop and bprop as nervanagpu/layers.py:26-277 does.
"""
from functools import reduce
from math import ceil
from operator import mul

import numpy as np

from . import _lib


def _prod(dims):
    return reduce(mul, dims, 1)


def _out_dim(x, f, pad, stride):
    return int(ceil(float(x - f + 1 + 2 * pad) / stride))


class Layer(object):
    """Base class: owns activations, deltas, weights and the SGD step."""

    def __init__(self, lib, dtype, N, dtypeU=None):
        self.N = N
        self.dtype = dtype
        self.dtypeU = dtype if dtypeU is None else dtypeU
        self.lib = lib
        self.flops = 0
        self.sizeI = self.sizeO = self.sizeF = 0
        self.weights = None
        self.fprop_in = None
        self.fprop_out = None
        self.bprop_out = None
        self.learning_rate = 0.0

    def init_activations(self):
        self.fprop_out = self.lib.empty(self.dimO, dtype=self.dtype)
        self.act_stats = self.lib.empty((self.dimO2[0], 1), dtype=np.float32)

    def init_deltas(self, shared=None):
        if shared is None:
            self.bprop_out = self.lib.empty(self.dimI, dtype=self.dtype)
        else:
            self.bprop_out = shared[0].share(self.dimI)
            shared.reverse()
        self.delta_stats = self.lib.empty((self.dimI2[0], 1), dtype=np.float32)

    def init_weights(self, loc=0.0, scale=0.1, shared=None, zeros=False, rng=None):
        if self.sizeF > 0:
            if zeros:
                self.weights = self.lib.zeros(self.dimF, dtype=self.dtype)
            else:
                rng = np.random if rng is None else rng
                self.weights = self.lib.array(rng.normal(loc, scale, self.dimF), dtype=self.dtype)
            if shared is None:
                self.updat_out = self.lib.empty(self.dimF, dtype=self.dtypeU)
            else:
                self.updat_out = shared.share(self.dimF, dtype=self.dtypeU)
            self.weight_stats = self.lib.empty((self.dimF2[0], 1), dtype=np.float32)

    def scale_weights(self, scale):
        mean = self.get_activation_mean()
        self.weights *= scale / mean

    def fprop(self, fprop_in, scale_weights=0):
        if self.fprop_in is None and fprop_in:
            self.fprop_in = fprop_in.reshape(self.dimI)
        return self.fprop_in

    def bprop(self, bprop_in):
        return bprop_in

    def bprop_relu(self, bprop_in):
        # the forward ReLU is fused into the conv / GEMM epilogue; its gradient is a mask
        bprop_in *= self.fprop_out > 0
        return bprop_in

    def grad_descent(self):
        self.weights += self.updat_out * self.learning_rate

    def _get_mean(self, ary, buf, shape):
        return float(self.lib.mean(abs(ary.reshape(shape)), partial=buf, out=buf[0:1, 0:1]).get()[0, 0])

    def _get_max(self, ary, buf, shape):
        return float(self.lib.max(abs(ary.reshape(shape)), partial=buf, out=buf[0:1, 0:1]).get()[0, 0])

    def get_activation_mean(self): return self._get_mean(self.fprop_out, self.act_stats, self.dimO2)
    def get_activation_max(self): return self._get_max(self.fprop_out, self.act_stats, self.dimO2)
    def get_delta_mean(self): return self._get_mean(self.bprop_out, self.delta_stats, self.dimI2)
    def get_delta_max(self): return self._get_max(self.bprop_out, self.delta_stats, self.dimI2)

    def get_update_mean(self):
        return self._get_mean(self.updat_out, self.weight_stats, self.dimF2) if self.sizeF > 0 else 0

    def get_update_max(self):
        return self._get_max(self.updat_out, self.weight_stats, self.dimF2) if self.sizeF > 0 else 0

    def get_weight_mean(self):
        return self._get_mean(self.weights, self.weight_stats, self.dimF2) if self.sizeF > 0 else 0

    def get_weight_max(self):
        return self._get_max(self.weights, self.weight_stats, self.dimF2) if self.sizeF > 0 else 0

    def fprop_stats(self):
        print("fprop:%10.5f mean %11.5f max %s" % (self.get_activation_mean(), self.get_activation_max(), self))

    def bprop_stats(self):
        if self.bprop_out is not None:
            print("bprop:%10.5f mean %11.5f max %s" % (self.get_delta_mean(), self.get_delta_max(), self))
        if self.weights is not None:
            up_mean, up_max = self.get_update_mean(), self.get_update_max()
            wt_mean, wt_max = self.get_weight_mean(), self.get_weight_max()
            print("updat:%10.5f mean %11.5f max %s" % (up_mean, up_max, self))
            print("weigh:%10.5f mean %11.5f max" % (wt_mean, wt_max))
            print("ratio:%10.5f mean %11.5f max" % (0.0001 * up_mean / wt_mean, 0.0001 * up_max / wt_max))

    @staticmethod
    def create(lib, conf, prev_layer, dtype):
        """Instantiate a layer from a config dict: {"layer": cls, "common": {...}, dtype: {...}, ...};
        N, C, H, W (or nIn) are propagated from the previous layer."""
        config = dict(conf)
        layer_type = config.pop("layer")
        if layer_type is Inception:
            # every branch is a chain of layers that starts on the container's input
            partitions = []
            for branch in config["partitions"]:
                chain, prev = [], prev_layer
                for inner in branch:
                    prev = Layer.create(lib, inner, prev, dtype)
                    chain.append(prev)
                partitions.append(chain)
            last = partitions[0][-1]
            return Inception(lib, dtype, partitions, prev_layer.N, prev_layer.K, sum(p[-1].K for p in partitions),
                             prev_layer.M, prev_layer.P, prev_layer.Q, last.M, last.P, last.Q)
        config["dtype"] = dtype
        config.update(config.pop(dtype, {}))
        config.update(config.pop("common", {}))
        if prev_layer is not None:
            config["N"] = prev_layer.N
            if layer_type is FullLayer:
                config["nIn"] = prev_layer.nOut
            elif layer_type is PoolLayer and type(prev_layer) is FullLayer:
                config["C"] = prev_layer.nOut
            else:
                config["C"] = prev_layer.K
                config["H"] = prev_layer.P
                config["W"] = prev_layer.Q
        for key in [k for k in config if type(k) is not str]:
            del config[key]
        return layer_type(lib, **config)


class DataLayer(Layer):
    def __init__(self, lib, dtype, N, C, D=1, H=1, W=1):
        super(DataLayer, self).__init__(lib, dtype, N)
        self.C = self.K = C
        self.M, self.P, self.Q = D, H, W
        self.DHW = (D, H, W)
        self.dimI = self.dimO = (C, D, H, W, N)
        self.dimI2 = self.dimO2 = (C * D * H * W, N)
        self.sizeO = self.sizeI = _prod(self.dimO)
        self.nOut = C * D * H * W

    def init_data(self, ary=None):
        if ary is None:
            self.fprop_out.fill(0)
        else:
            self.fprop_out.set(ary)

    def init_deltas(self, shared=None):
        pass

    def init_weights(self, loc=0.0, scale=0.1, shared=None, zeros=False, rng=None):
        pass

    def fprop(self, fprop_in, scale_weights=0):
        return self.fprop_out

    def __str__(self):
        return "DataLayer: NCK: (%d, %d, %d) DHW:%s" % (self.N, self.C, self.K, self.DHW)


class FullLayer(Layer):
    def __init__(self, lib, dtype, N, nIn, nOut):
        super(FullLayer, self).__init__(lib, dtype, N)
        self.nIn, self.nOut = nIn, nOut
        self.flops = N * nIn * nOut * 2.0
        self.dimI = self.dimI2 = (nIn, N)
        self.dimO = self.dimO2 = (nOut, N)
        self.dimF = self.dimF2 = (nOut, nIn)
        self.sizeI, self.sizeO, self.sizeF = nIn * N, nOut * N, nIn * nOut

    def fprop(self, fprop_in, scale_weights=0):
        fprop_in = super(FullLayer, self).fprop(fprop_in)
        self.lib.dot(self.weights, fprop_in, self.fprop_out, relu=True)
        if scale_weights:
            self.scale_weights(scale_weights)
            self.fprop(fprop_in)
        return self.fprop_out

    def bprop(self, bprop_in):
        self.bprop_relu(bprop_in)
        self.lib.dot(self.weights.T, bprop_in, self.bprop_out)
        self.lib.dot(bprop_in, self.fprop_in.T, self.updat_out)
        self.grad_descent()
        return self.bprop_out

    def __str__(self):
        return "FullLayer: N, nIn, nOut: (%d, %d, %d)" % (self.N, self.nIn, self.nOut)


class ConvLayer(Layer):
    """Convolution parameters: I (C,D,H,W,N) * F (C,T,R,S,K) -> O (K,M,P,Q,N)."""

    def __init__(self, lib, dtype, N, C, K, D=1, H=1, W=1, T=1, R=1, S=1, pad_d=0, pad_h=0, pad_w=0,
                 str_d=1, str_h=1, str_w=1, grid_P=0, grid_Q=0, update_size=None):
        # weight gradients are produced in fp32 (nervanagpu/layers.py:289)
        super(ConvLayer, self).__init__(lib, dtype, N, np.float32)
        assert N % 8 == 0, "N dim must be multiple of 8"
        assert K % 8 == 0, "K dim must be multiple of 8"

        M = _out_dim(D, T, pad_d, str_d)
        P = _out_dim(H, R, pad_h, str_h)
        Q = _out_dim(W, S, pad_w, str_w)
        self.C, self.K, self.M, self.P, self.Q = C, K, M, P, Q
        self.NCK = (N, C, K)
        self.TRS = (T, R, S)
        self.DHW = (D, H, W)
        self.MPQ = (M, P, Q)
        self.padding = (pad_d, pad_h, pad_w)
        self.strides = (str_d, str_h, str_w)
        self.dimI = (C, D, H, W, N)
        self.dimF = (C, T, R, S, K)
        self.dimFb = (K, T, R, S, C)
        self.dimO = (K, M, P, Q, N)
        self.dimI2 = (C * D * H * W, N)
        self.dimF2 = (C * T * R * S, K)
        self.dimF2t = (K, C * T * R * S)
        self.dimO2 = (K * M * P * Q, N)
        self.sizeI = _prod(self.dimI)
        self.sizeF = _prod(self.dimF)
        self.sizeO = _prod(self.dimO)
        self.nOut = M * P * Q * K
        # flops of one pass, padded taps counted (nervanagpu/layers.py:422)
        self.flops = M * P * Q * K * N * C * T * R * S * 2.0
        self.desc = _lib.ConvDesc(N, C, K, D, H, W, T, R, S, pad_d, pad_h, pad_w, str_d, str_h, str_w)
        self.path = _lib.NG_PATH_AUTO

    def fprop(self, fprop_in, scale_weights=0):
        fprop_in = super(ConvLayer, self).fprop(fprop_in)
        self.lib.fprop_conv(self, fprop_in, self.weights, self.fprop_out, relu=True)
        if scale_weights:
            self.scale_weights(scale_weights)
            self.fprop(fprop_in)
        return self.fprop_out

    def bprop(self, bprop_in):
        self.bprop_relu(bprop_in)
        if self.bprop_out is not None:
            self.lib.bprop_conv(self, self.weights, bprop_in, self.bprop_out)
        self.lib.update_conv(self, self.fprop_in, bprop_in, self.updat_out)
        self.grad_descent()
        return self.bprop_out

    def __str__(self):
        return ("ConvLayer: NCK: (%d, %d, %d) DHW:%s TRS:%s MPQ:%s" %
                (self.N, self.C, self.K, self.DHW, self.TRS, self.MPQ))


class DeconvLayer(ConvLayer):
    """Transposed convolution: fprop is the conv backward pass, bprop the conv forward pass
    (nervanagpu/layers.py:509-537). Built from the output size P, Q of the equivalent conv."""

    def __init__(self, lib, dtype, N, C, K, P, Q, R=1, S=1, pad_d=0, pad_h=0, pad_w=0, str_d=1, str_h=1, str_w=1,
                 grid_P=0, grid_Q=0, update_size=None):
        H = (P - 1) * str_h - 2 * pad_h + R
        W = (Q - 1) * str_w - 2 * pad_w + S
        super(DeconvLayer, self).__init__(lib, dtype, N, C, K, 1, H, W, 1, R, S, pad_d, pad_h, pad_w,
                                          str_d, str_h, str_w, grid_P, grid_Q, update_size)
        self.nOut = reduce(mul, self.DHW, 1) * C
        self.H, self.W = H, W

    def fprop(self, fprop_in, scale_weights=0):
        if self.fprop_in is None and fprop_in:
            self.fprop_in = fprop_in.reshape(self.dimO)
        self.lib.bprop_conv(self, self.weights, self.fprop_in, self.fprop_out)
        return self.fprop_out

    def init_activations(self):
        self.fprop_out = self.lib.empty(self.dimI, dtype=self.dtype)
        self.act_stats = self.lib.empty((self.dimI2[0], 1), dtype=np.float32)

    def bprop(self, bprop_in):
        if self.bprop_out is not None:
            self.lib.fprop_conv(self, bprop_in, self.weights, self.bprop_out)
        self.lib.update_conv(self, bprop_in, self.fprop_in, self.updat_out)
        self.grad_descent()
        return self.bprop_out

    def __str__(self):
        return ("DeconvLayer: NCK: (%d, %d, %d) DHW:%s TRS:%s MPQ:%s" %
                (self.N, self.C, self.K, self.DHW, self.TRS, self.MPQ))


class PoolLayer(Layer):
    """Pooling parameters: windows (J,T,R,S) over (C,D,H,W); op is "max", "avg" or "l2". (The
    reference accepts all three but launches its max kernel for every op,
    nervanagpu/nervanagpu.py:797, and defines avg / l2 in numpy only, benchmarks/pool_test.py:141-146;
    here each runs its own kernel.)"""

    def __init__(self, lib, dtype, op, N, C, D=1, H=1, W=1, J=1, T=1, R=1, S=1, pad_j=0, pad_d=0, pad_h=0,
                 pad_w=0, str_j=None, str_d=None, str_h=None, str_w=None):
        super(PoolLayer, self).__init__(lib, dtype, N)
        if str_j is None: str_j = J
        if str_d is None: str_d = T
        if str_h is None: str_h = R
        if str_w is None: str_w = S
        if str_j < J or str_d < T or str_h < R or str_w < S:
            self.overlap = (ceil(float(J) / str_j) * ceil(float(T) / str_d) *
                            ceil(float(R) / str_h) * ceil(float(S) / str_w))
        else:
            self.overlap = 0.0
        K = _out_dim(C, J, pad_j, str_j)
        M = _out_dim(D, T, pad_d, str_d)
        P = _out_dim(H, R, pad_h, str_h)
        Q = _out_dim(W, S, pad_w, str_w)
        self.op = op
        self.C, self.K, self.M, self.P, self.Q = C, K, M, P, Q
        self.JTRS = (J, T, R, S)
        self.DHW = (D, H, W)
        self.MPQ = (M, P, Q)
        self.padding = (pad_j, pad_d, pad_h, pad_w)
        self.strides = (str_j, str_d, str_h, str_w)
        self.dimI = (C, D, H, W, N)
        self.dimO = (K, M, P, Q, N)
        self.dimF2 = None
        self.dimI2 = (C * D * H * W, N)
        self.dimO2 = (K * M * P * Q, N)
        self.sizeI = _prod(self.dimI)
        self.sizeO = _prod(self.dimO)
        self.nOut = M * P * Q * K
        self.desc = _lib.PoolDesc(N, C, D, H, W, J, T, R, S, pad_j, pad_d, pad_h, pad_w,
                                  str_j, str_d, str_h, str_w)

    def fprop(self, fprop_in, scale_weights=0):
        fprop_in = super(PoolLayer, self).fprop(fprop_in)
        self.lib.fprop_pool(self, fprop_in, self.fprop_out)
        return self.fprop_out

    def bprop(self, bprop_in):
        self.lib.bprop_pool(self, self.fprop_in, bprop_in, self.bprop_out)
        return self.bprop_out

    def __str__(self):
        return ("PoolLayer: NCK: (%d, %d, %d) DHW:%s JTRS:%s MPQ:%s op: %s " %
                (self.N, self.C, self.K, self.DHW, self.JTRS, self.MPQ, self.op))


class Inception(Layer):
    """Parallel branches over one input whose outputs are concatenated along the feature-map
    dimension (nervanagpu/layers.py:643-755). `partitions` is a list of branches, each a list of
    layers already created on the container's input shape.

    The output of every branch's last layer is a channel slice of the container's output, so the
    concatenation costs nothing. On the way back each branch takes its slice of the incoming
    deltas; the branches' input deltas are summed: the first branch writes the container's delta
    buffer, the others write a scratch buffer that is then added to it. (The reference lets every
    branch overwrite the same buffer and leaves the sum as a TODO, nervanagpu/layers.py:737.)
    """

    def __init__(self, lib, dtype, partitions, N, C, K, D=1, H=1, W=1, M=1, P=1, Q=1):
        super(Inception, self).__init__(lib, dtype, N)
        self.partitions = [list(part) for part in partitions]
        self.C, self.K, self.M, self.P, self.Q = C, K, M, P, Q
        self.NCK = (N, C, K)
        self.DHW = (D, H, W)
        self.MPQ = (M, P, Q)
        self.dimI = (C, D, H, W, N)
        self.dimO = (K, M, P, Q, N)
        self.dimI2 = (C * D * H * W, N)
        self.dimO2 = (K * M * P * Q, N)
        self.sizeI = _prod(self.dimI)
        self.sizeO = _prod(self.dimO)
        self.nOut = M * P * Q * K
        inner = [layer for part in self.partitions for layer in part]
        assert sum(part[-1].K for part in self.partitions) == K
        assert all(part[-1].MPQ == self.MPQ for part in self.partitions), "branches must end on one map size"
        self.flops = sum(layer.flops for layer in inner)
        widest = max(inner, key=lambda layer: layer.sizeF)
        self.sizeF = widest.sizeF
        if self.sizeF:
            self.dimF = widest.dimF

    def init_activations(self):
        super(Inception, self).init_activations()
        k0 = 0
        for part in self.partitions:
            for layer in part[:-1]:
                layer.init_activations()
            last = part[-1]
            last.fprop_out = self.fprop_out[k0:k0 + last.K]
            last.act_stats = self.lib.empty((last.dimO2[0], 1), dtype=np.float32)
            k0 += last.K

    def init_deltas(self, shared=None):
        super(Inception, self).init_deltas(shared)
        self._branch_delta = self.lib.empty(self.dimI, dtype=self.dtype) if len(self.partitions) > 1 else None
        for b, part in enumerate(self.partitions):
            part[0].bprop_out = self.bprop_out if b == 0 else self._branch_delta
            part[0].delta_stats = self.delta_stats
            for layer in part[1:]:
                layer.init_deltas()

    def init_weights(self, loc=0.0, scale=0.1, shared=None, zeros=False, rng=None):
        for part in self.partitions:
            for layer in part:
                layer.init_weights(loc, scale, shared, zeros, rng)

    def fprop(self, fprop_in, scale_weights=0):
        fprop_in = super(Inception, self).fprop(fprop_in)
        for part in self.partitions:
            x = fprop_in
            for layer in part:
                x = layer.fprop(x, scale_weights)
        return self.fprop_out

    def bprop(self, bprop_in):
        k0 = 0
        for b, part in enumerate(self.partitions):
            delta = bprop_in.reshape(self.dimO)[k0:k0 + part[-1].K]
            k0 += part[-1].K
            for layer in part[::-1]:
                delta = layer.bprop(delta)
            if b > 0 and self.bprop_out is not None:
                self.bprop_out[:] = self.bprop_out + self._branch_delta
        return self.bprop_out

    def fprop_stats(self):
        for part in self.partitions:
            for layer in part:
                layer.fprop_stats()

    def bprop_stats(self):
        for part in self.partitions[::-1]:
            for layer in part[::-1]:
                layer.bprop_stats()

    def __str__(self):
        lines = ["Inception: NCK: (%d, %d, %d) DHW:%s MPQ:%s" % (self.N, self.C, self.K, self.DHW, self.MPQ)]
        for i, part in enumerate(self.partitions):
            lines.append("  Part%d:" % (i + 1))
            lines.extend("    %s" % layer for layer in part)
        return "\n".join(lines)
