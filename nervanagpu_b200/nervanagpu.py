"""Host-side API: the NervanaGPU factory, GPUTensor and the lazy OpTreeNode.

Same names, arguments and error behaviour as the reference's nervanagpu/nervanagpu.py
(GPUTensor :30-466, NervanaGPU :469-1224, OpTreeNode :1227-1319), with PyCUDA replaced by the
ctypes C ABI of libnervana_b200.so. Strides are in elements, tensors are row-major, views keep
their base alive, `.T` flips `is_trans`, and arithmetic on tensors builds an op tree that is
collapsed into one generated kernel on assignment.
"""
import ctypes
from functools import reduce
from operator import mul
import struct
import weakref

import numpy as np

from . import _lib
from .float_ew import call_compound_kernel
from .layers import ConvLayer, DeconvLayer, PoolLayer

_none_slice = slice(None, None, None)
_DTYPES = (np.float16, np.float32, np.uint8, np.int8, np.uint16, np.int16, np.uint32, np.int32)


def _contiguous_strides(shape):
    """Row-major strides in elements (not bytes)."""
    if not shape:
        return ()
    strides = [1]
    for s in shape[:0:-1]:
        strides.append(strides[-1] * s)
    return tuple(strides[::-1])


class DeviceAllocation(object):
    """Owning handle of one ng_malloc block; int() gives the device address."""

    def __init__(self, nbytes):
        lib = _lib.init()
        ptr = ctypes.c_void_p()
        _lib.check(lib.ng_malloc(ctypes.byref(ptr), nbytes))
        self.ptr = ptr.value or 0
        self.nbytes = nbytes
        self._finalizer = weakref.finalize(self, DeviceAllocation._release, lib, self.ptr)

    @staticmethod
    def _release(lib, ptr):
        try:
            lib.ng_free(ptr)
        except Exception:
            pass

    def free(self):
        self._finalizer()

    def __int__(self):
        return self.ptr

    __index__ = __int__


def mem_alloc(nbytes):
    return DeviceAllocation(nbytes)


class GPUTensor(object):

    def __init__(self, backend, shape, dtype=np.float16, allocator=mem_alloc, base=None, gpudata=None,
                 strides=None, take_array=None, is_trans=False, name=None, rounding=0):
        assert dtype in _DTYPES or np.dtype(dtype).type in _DTYPES
        dtype = np.dtype(dtype)
        try:
            size = 1
            for dim in shape:
                size *= dim
            shape = tuple(int(d) for d in shape)
        except TypeError:
            assert isinstance(shape, (int, np.integer))
            size = shape
            shape = (int(shape),)
        size = int(size)

        self.strides = _contiguous_strides(shape) if strides is None else tuple(strides)
        self.backend = backend
        self.base = base
        self.shape = shape
        self.size = size
        self.dtype = dtype
        self.nbytes = dtype.itemsize * size
        self.allocator = allocator
        self.take_array = take_array
        self.is_trans = is_trans
        self.name = name
        self.rounding = rounding
        self.kahan_count = 0
        self.kahan_reset = 0

        if gpudata is None:
            self.gpudata = allocator(self.nbytes) if size else None
            assert base is None
        else:
            self.gpudata = gpudata

    def __str__(self):
        return ("Array(0x%x) name:%s dtype:%s shape:%s strides:%s  is_trans:%s" %
                (self.ptr, self.name, self.dtype, self.shape, self.strides, self.is_trans))

    __repr__ = __str__

    def __int__(self):
        return self.ptr

    @property
    def ptr(self):
        return 0 if self.gpudata is None else int(self.gpudata)

    def __len__(self):
        return self.shape[0] if len(self.shape) else 0

    # tensors are compared by identity when used as dict keys (operators build op trees)
    def __hash__(self):
        return id(self)

    @property
    def is_contiguous(self):
        return not self.take_array and self.strides == _contiguous_strides(self.shape)

    @property
    def __cuda_array_interface__(self):
        assert self.is_contiguous
        return {"shape": self.shape, "typestr": self.dtype.str, "data": (self.ptr, False), "version": 2}

    def set(self, ary):
        """Copy a host array to the device; the tensor must be contiguous."""
        assert ary.size == self.size
        assert self.is_contiguous, "Array in set() must be contiguous"
        if ary.dtype != self.dtype:
            ary = ary.astype(self.dtype)
        ary = np.ascontiguousarray(ary)
        if self.size:
            lib = _lib.init()
            _lib.check(lib.ng_memcpy_h2d_async(self.ptr, ary.ctypes.data, self.nbytes, self.backend.stream))
            # pageable source: the call has consumed `ary` when it returns
        return self

    def get(self, stream=None):
        """Copy the device array to a new host array (synchronous)."""
        assert self.is_contiguous, "Array in get() must be contiguous"
        ary = np.empty(self.shape, self.dtype)
        if self.size:
            lib = _lib.init()
            if stream is None:
                stream = self.backend.stream     # ordered after the work queued on the backend's stream
            _lib.check(lib.ng_memcpy_d2h_async(ary.ctypes.data, self.ptr, self.nbytes, stream))
            _lib.check(lib.ng_stream_sync(stream))
        return ary

    def asnumpyarray(self):
        return self.get()

    def take(self, indices, axis, out=None):
        view = self[(_none_slice, indices)] if axis == 1 else self[(indices, _none_slice)]
        if out:
            return out._assign(view)
        return view

    def __getitem__(self, index):
        """Sliced / fancy-indexed view."""
        if not isinstance(index, tuple):
            if isinstance(index, slice) and index == _none_slice:
                return self
            index = (index,)

        new_shape, new_strides = [], []
        new_offset = 0
        seen_ellipsis = False
        take_array = None
        index_axis = array_axis = 0
        while index_axis < len(index):
            entry = index[index_axis]
            if array_axis > len(self.shape):
                raise IndexError("too many axes in index")

            if isinstance(entry, slice):
                start, stop, step = entry.indices(self.shape[array_axis])
                array_stride = self.strides[array_axis]
                new_shape.append(-((start - stop) // step))
                new_strides.append(step * array_stride)
                new_offset += array_stride * start * self.dtype.itemsize
                index_axis += 1
                array_axis += 1

            elif isinstance(entry, (GPUTensor, np.ndarray, list, tuple)):
                if isinstance(entry, (list, tuple)):
                    entry = np.array(entry, dtype=np.int32)
                if isinstance(entry, np.ndarray):
                    entry = self.__class__(self.backend, entry.shape, dtype=np.int32).set(entry)
                size = max(entry.shape)
                if size != entry.size:
                    raise IndexError("Fancy indexing only currently supported for dim > 1 in a single dimension.")
                if take_array is not None:
                    raise IndexError("Fancy indexing only currently supported for one axis at a time.")
                if entry.dtype.type is not np.int32:
                    raise IndexError("Fancy indexing only currently supported with int32 types.")
                take_array = (entry, array_axis)
                new_shape.append(size)
                new_strides.append(self.strides[array_axis])
                index_axis += 1
                array_axis += 1

            elif isinstance(entry, (int, np.integer)):
                extent = self.shape[array_axis]
                if entry < 0:
                    entry += extent
                if not (0 <= entry < extent):
                    raise IndexError("subindex in axis %d out of range" % index_axis)
                new_offset += self.strides[array_axis] * int(entry) * self.dtype.itemsize
                index_axis += 1
                array_axis += 1

            elif entry is Ellipsis:
                index_axis += 1
                remaining = len(index) - index_axis
                new_array_axis = len(self.shape) - remaining
                if new_array_axis < array_axis:
                    raise IndexError("invalid use of ellipsis in index")
                while array_axis < new_array_axis:
                    new_shape.append(self.shape[array_axis])
                    new_strides.append(self.strides[array_axis])
                    array_axis += 1
                if seen_ellipsis:
                    raise IndexError("more than one ellipsis not allowed in index")
                seen_ellipsis = True
            else:
                raise IndexError("invalid subindex in axis %d" % index_axis)

        while array_axis < len(self.shape):
            new_shape.append(self.shape[array_axis])
            new_strides.append(self.strides[array_axis])
            array_axis += 1

        return self.__class__(backend=self.backend, shape=tuple(new_shape), dtype=self.dtype,
                              allocator=self.allocator, base=self, gpudata=self.ptr + new_offset,
                              strides=new_strides, take_array=take_array, name=self.name,
                              rounding=self.rounding)

    def _assign(self, value):
        stream = self.backend.stream
        if isinstance(value, (int, float)):
            if self.is_contiguous:
                # contiguous fill: memset of the value's bit pattern
                lib = _lib.init()
                bits = np.array(value).astype(self.dtype).tobytes()
                if not self.size:
                    pass
                elif self.dtype.itemsize == 1:
                    _lib.check(lib.ng_memset_d8_async(self.ptr, struct.unpack("B", bits)[0], self.size, stream))
                elif self.dtype.itemsize == 2:
                    _lib.check(lib.ng_memset_d16_async(self.ptr, struct.unpack("H", bits)[0], self.size, stream))
                else:
                    _lib.check(lib.ng_memset_d32_async(self.ptr, struct.unpack("I", bits)[0], self.size, stream))
            else:
                OpTreeNode.build("assign", self, value)

        elif isinstance(value, GPUTensor):
            if self.is_contiguous and value.is_contiguous and self.dtype == value.dtype and not value.is_trans:
                if self.size:
                    _lib.check(_lib.init().ng_memcpy_d2d_async(self.ptr, value.ptr, self.nbytes, stream))
            else:
                OpTreeNode.build("assign", self, value)

        elif isinstance(value, OpTreeNode):
            OpTreeNode.build("assign", self, value)

        elif isinstance(value, np.ndarray):
            self.set(value)

        else:
            raise TypeError("Invalid type for assignment: %s" % type(value))
        return self

    def __setitem__(self, index, value):
        self.__getitem__(index)._assign(value)

    def fill(self, value):
        return self._assign(value)

    def copy(self, a):
        return self._assign(a)

    def copy_from(self, a):
        return self.set(a)

    def reshape(self, *shape):
        if isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        if shape == self.shape:
            return self
        size = reduce(mul, shape, 1)
        if size != self.size:
            raise ValueError("total size of new array must be unchanged")
        if not self.is_contiguous:
            raise TypeError("reshaping of non-contigous arrays is not yet supported")
        return self.__class__(backend=self.backend, shape=shape, dtype=self.dtype, allocator=self.allocator,
                              base=self, gpudata=self.gpudata, strides=_contiguous_strides(shape),
                              name=self.name, rounding=self.rounding)

    def share(self, shape, dtype=None, name=None):
        """View of the same memory with another (not larger) shape; for scratch reuse."""
        size = reduce(mul, shape, 1)
        if size > self.size:
            raise ValueError("total size of new array must <= size of parent")
        if not self.is_contiguous:
            raise TypeError("sharing of non-contigous arrays is not yet supported")
        dtype = self.dtype if dtype is None else np.dtype(dtype)
        return self.__class__(backend=self.backend, shape=shape, dtype=dtype, allocator=self.allocator,
                              base=self, gpudata=self.gpudata, strides=_contiguous_strides(shape),
                              name=name, rounding=self.rounding)

    @property
    def T(self):
        if len(self.shape) <= 2:
            shape = self.shape[::-1]
            strides = self.strides[::-1]
        else:
            # batched dot: keep the outer dimension, reverse the inner two
            shape = list(self.shape[::-1])
            strides = list(self.strides[::-1])
            shape = tuple(shape[-1:] + shape[:-1])
            strides = tuple(strides[-1:] + strides[:-1])
        return self.__class__(backend=self.backend, shape=shape, dtype=self.dtype, allocator=self.allocator,
                              base=self, gpudata=self.gpudata, strides=strides,
                              is_trans=not self.is_trans, name=self.name, rounding=self.rounding)

    def transpose(self, out=None):
        if out:
            return OpTreeNode.build("assign", out, self.T)
        return self.T

    def __add__(self, other): return OpTreeNode.build("add", self, other)
    def __sub__(self, other): return OpTreeNode.build("sub", self, other)
    def __mul__(self, other): return OpTreeNode.build("mul", self, other)
    def __div__(self, other): return OpTreeNode.build("div", self, other)
    def __truediv__(self, other): return OpTreeNode.build("div", self, other)
    def __pow__(self, other): return OpTreeNode.build("pow", self, other)
    def __radd__(self, other): return OpTreeNode.build("add", other, self)
    def __rsub__(self, other): return OpTreeNode.build("sub", other, self)
    def __rmul__(self, other): return OpTreeNode.build("mul", other, self)
    def __rdiv__(self, other): return OpTreeNode.build("div", other, self)
    def __rtruediv__(self, other): return OpTreeNode.build("div", other, self)
    def __rpow__(self, other): return OpTreeNode.build("pow", other, self)
    def __eq__(self, other): return OpTreeNode.build("eq", self, other)
    def __ne__(self, other): return OpTreeNode.build("ne", self, other)
    def __lt__(self, other): return OpTreeNode.build("lt", self, other)
    def __le__(self, other): return OpTreeNode.build("le", self, other)
    def __gt__(self, other): return OpTreeNode.build("gt", self, other)
    def __ge__(self, other): return OpTreeNode.build("ge", self, other)
    def __abs__(self): return OpTreeNode.build("abs", self, None)
    def __neg__(self): return OpTreeNode.build("neg", self, None)

    def __iadd__(self, other): return OpTreeNode.build("add", self, other, out=self)
    def __isub__(self, other): return OpTreeNode.build("sub", self, other, out=self)
    def __imul__(self, other): return OpTreeNode.build("mul", self, other, out=self)
    def __idiv__(self, other): return OpTreeNode.build("div", self, other, out=self)
    def __itruediv__(self, other): return OpTreeNode.build("div", self, other, out=self)
    def __ipow__(self, other): return OpTreeNode.build("pow", self, other, out=self)


class RandState(object):
    """Position in the Philox stream used by stochastic rounding and rand(): a fixed seed and a
    per-launch offset (the reference keeps a 2048*32-word LFSR pool instead,
    nervanagpu/nervanagpu.py:1337-1346; with Philox, reruns with the same seed repeat exactly)."""

    def __init__(self, seed=0xB200):
        self.seed = int(seed) & 0xFFFFFFFFFFFFFFFF
        self.offset = 0

    def next_offset(self):
        off = self.offset
        self.offset = (self.offset + 1) & 0xFFFFFFFF
        return off


class RecordedSequence(object):
    """Device work recorded by NervanaGPU.capture(); launch() queues all of it with one call.
    A replay repeats the recorded pointers, scalars and random offsets exactly."""

    def __init__(self, backend, handle):
        self.backend = backend
        self.handle = handle

    def launch(self):
        _lib.check(self.backend.lib.ng_graph_launch(self.handle, self.backend.stream))

    def release(self):
        if self.handle is not None:
            _lib.check(self.backend.lib.ng_graph_destroy(self.handle))
            self.handle = None

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


class NervanaGPU(object):

    def __init__(self, stochastic_round=False, bench=False, cubin_path=None, scratch_size=9 * 1024 * 1024,
                 default_dtype=np.float16, seed=0xB200, device=None):
        """Factory for GPUTensors and entry point of every device operation.

        stochastic_round: mantissa bits to round to stochastically (True = 10), 0/False = off.
        bench: truthy prints timing for GEMM / conv / pool calls.
        cubin_path, scratch_size: accepted for compatibility; kernels live in the shared library
        and scratch memory is managed by it.
        """
        if stochastic_round:
            if stochastic_round is True:
                stochastic_round = 10
        else:
            stochastic_round = 0
        self.scratch_size = scratch_size
        self.round_mode = stochastic_round
        self.cubin_path = cubin_path
        self.bench = bench
        self.stream = None
        self.default_dtype = default_dtype
        self.rand_state = RandState(seed)
        self.lib = _lib.init(device)
        self._events = None

    # ---- allocation helpers --------------------------------------------------------------
    def empty(self, shape, dtype=None, name=None, allocator=mem_alloc):
        dtype = self.default_dtype if dtype is None else dtype
        return GPUTensor(self, shape, dtype, allocator=allocator, name=name, rounding=self.round_mode)

    def array(self, ary, dtype=None, name=None, allocator=mem_alloc):
        dtype = self.default_dtype if dtype is None else dtype
        return GPUTensor(self, ary.shape, dtype, allocator=allocator, name=name,
                         rounding=self.round_mode).set(ary)

    def zeros(self, shape, dtype=None, name=None, allocator=mem_alloc):
        dtype = self.default_dtype if dtype is None else dtype
        return GPUTensor(self, shape, dtype, allocator=allocator, name=name,
                         rounding=self.round_mode)._assign(0)

    def ones(self, shape, dtype=None, name=None, allocator=mem_alloc):
        dtype = self.default_dtype if dtype is None else dtype
        return GPUTensor(self, shape, dtype, allocator, name=name, rounding=self.round_mode)._assign(1)

    def empty_like(self, other_ary, name=None):
        return GPUTensor(self, other_ary.shape, other_ary.dtype, other_ary.allocator, name=name,
                         rounding=self.round_mode)

    def zeros_like(self, other_ary, name=None):
        return GPUTensor(self, other_ary.shape, other_ary.dtype, other_ary.allocator, name=name,
                         rounding=self.round_mode)._assign(0)

    def synchronize(self):
        _lib.check(self.lib.ng_sync())

    # ---- streams and recorded sequences --------------------------------------------------
    def new_stream(self):
        """A new stream handle; assign it to `self.stream` to queue all later work on it."""
        s = ctypes.c_void_p()
        _lib.check(self.lib.ng_stream_create(ctypes.byref(s)))
        return s

    def capture(self, fn):
        """Record the device work `fn()` queues on `self.stream` (which must be a stream from
        new_stream, not the default one) and return a RecordedSequence whose launch() replays it
        with one host call. `fn` must have run once before with the same tensors, so that scratch
        memory has its final size and generated kernels exist. No pycuda-era counterpart: the
        reference launches every kernel from Python (nervanagpu/nervanagpu.py:705-729)."""
        _lib.check(self.lib.ng_graph_capture_begin(self.stream))
        graph = ctypes.c_void_p()
        try:
            fn()
        finally:
            rc = self.lib.ng_graph_capture_end(self.stream, ctypes.byref(graph))
        _lib.check(rc)
        return RecordedSequence(self, graph)

    # ---- timing --------------------------------------------------------------------------
    def _get_events(self):
        if self._events is None:
            a, b = ctypes.c_void_p(), ctypes.c_void_p()
            _lib.check(self.lib.ng_event_create(ctypes.byref(a)))
            _lib.check(self.lib.ng_event_create(ctypes.byref(b)))
            self._events = (a, b)
        return self._events

    def _timed(self, launch, repeat, pre=None):
        """Warm-up max(repeat//10, 1) launches when repeat > 1, then `repeat` launches between two
        events (as nervanagpu/nervanagpu.py:705-729). Returns msecs per launch or None."""
        if repeat > 1:
            for _ in range(max(repeat // 10, 1)):
                launch()
        timing = self.bench or repeat > 1
        if timing:
            start, end = self._get_events()
            _lib.check(self.lib.ng_event_record(start, self.stream))
        for _ in range(repeat):
            if pre is not None:
                pre()
            launch()
        if timing:
            _lib.check(self.lib.ng_event_record(end, self.stream))
            _lib.check(self.lib.ng_event_sync(end))
            ms = ctypes.c_float()
            _lib.check(self.lib.ng_event_elapsed_ms(start, end, ctypes.byref(ms)))
            return ms.value / repeat
        return None

    # ---- convolution ---------------------------------------------------------------------
    def conv_layer(self, dtype, N, C, K, D=1, H=1, W=1, T=1, R=1, S=1, pad_d=0, pad_h=0, pad_w=0,
                   str_d=1, str_h=1, str_w=1, grid_P=0, grid_Q=0, update_size=None):
        """Create a ConvLayer parameter object (dimensions as nervanagpu/nervanagpu.py:540-589).
        grid_P, grid_Q and update_size tuned the reference's Maxwell kernels; they are accepted
        and ignored (work distribution is chosen by the library)."""
        return ConvLayer(self, dtype, N, C, K, D, H, W, T, R, S, pad_d, pad_h, pad_w, str_d, str_h, str_w,
                         grid_P, grid_Q, update_size)

    def deconv_layer(self, dtype, N, C, K, P, Q, R=1, S=1, pad_d=0, pad_h=0, pad_w=0, str_d=1, str_h=1, str_w=1,
                     grid_P=0, grid_Q=0, update_size=None):
        return DeconvLayer(self, dtype, N, C, K, P, Q, R, S, pad_d, pad_h, pad_w, str_d, str_h, str_w,
                           grid_P, grid_Q, update_size)

    def fprop_conv(self, layer, I, F, O, alpha=1.0, relu=False, repeat=1):
        assert layer.sizeI == I.size
        assert layer.sizeF == F.size
        assert layer.sizeO == O.size
        return self._execute_conv(layer, "fprop", I, F, O, alpha, relu, repeat)

    def bprop_conv(self, layer, F, E, grad_I, alpha=1.0, repeat=1):
        assert layer.sizeF == F.size
        assert layer.sizeO == E.size
        assert layer.sizeI == grad_I.size
        return self._execute_conv(layer, "bprop", E, F, grad_I, alpha, False, repeat)

    def update_conv(self, layer, I, E, grad_F, alpha=1.0, repeat=1):
        assert layer.sizeI == I.size
        assert layer.sizeO == E.size
        assert layer.sizeF == grad_F.size
        return self._execute_conv(layer, "updat", I, E, grad_F, alpha, False, repeat)

    def _execute_conv(self, layer, op, A, B, C, alpha, relu, repeat):
        assert A.dtype == B.dtype
        if A.dtype.type is not np.float16:
            raise TypeError("Only fp16 convolution is supported (fp32 sconv kernels are not part of this library).")
        desc = ctypes.byref(layer.desc)
        path = getattr(layer, "path", _lib.NG_PATH_AUTO)
        lib, stream = self.lib, self.stream
        if op == "fprop":
            assert C.dtype.type is np.float16
            launch = lambda: _lib.check(lib.ng_conv_fprop(desc, A.ptr, B.ptr, C.ptr, alpha, int(bool(relu)), path, stream))
        elif op == "bprop":
            assert C.dtype.type is np.float16
            launch = lambda: _lib.check(lib.ng_conv_bprop(desc, B.ptr, A.ptr, C.ptr, alpha, path, stream))
        else:
            if C.dtype.type not in (np.float32, np.float16):
                raise TypeError("update_conv output must be fp32 or fp16")
            out_f32 = int(C.dtype.type is np.float32)
            launch = lambda: _lib.check(lib.ng_conv_update(desc, A.ptr, B.ptr, C.ptr, out_f32, alpha, path, stream))
        msecs = self._timed(launch, repeat)
        if msecs is not None:
            gflops = layer.flops / (msecs * 1000000.0)
            print("%7.3f msecs %8.3f gflops %6.0f (%s: %s)" % (msecs, gflops, layer.flops / 1000000.0, op, layer))
            return msecs, gflops
        return 0, 0

    # ---- pooling -------------------------------------------------------------------------
    def pool_layer(self, dtype, op, N, C, D=1, H=1, W=1, J=1, T=1, R=1, S=1, pad_j=0, pad_d=0, pad_h=0, pad_w=0,
                   str_j=None, str_d=None, str_h=None, str_w=None):
        """Create a PoolLayer parameter object (nervanagpu/nervanagpu.py:736-771). Strides default
        to the window (non-overlapping)."""
        if str_j is None: str_j = J
        if str_d is None: str_d = T
        if str_h is None: str_h = R
        if str_w is None: str_w = S
        return PoolLayer(self, dtype, op, N, C, D, H, W, J, T, R, S, pad_j, pad_d, pad_h, pad_w,
                         str_j, str_d, str_h, str_w)

    def pool_argmax_bytes(self, layer, dtype=np.float16):
        """Size of the buffer fprop_pool(..., argmax=) fills, or 0 when this layer has no such path."""
        if getattr(layer, "op", "max") != "max":
            return 0
        n = ctypes.c_size_t()
        _lib.check(self.lib.ng_pool_argmax_bytes(ctypes.byref(layer.desc), np.dtype(dtype).itemsize, ctypes.byref(n)))
        return n.value

    def fprop_pool(self, layer, I, O, repeat=1, argmax=None):
        """argmax: optional uint8 tensor of pool_argmax_bytes(layer) elements that receives each
        window's argmax, for bprop_pool(..., argmax=) (an extension: the reference's backward
        kernel rescans the windows, nervanagpu/nervanagpu.py:780-787)."""
        assert layer.sizeI == I.size
        assert layer.sizeO == O.size
        return self._execute_pool(layer, I, O, None, 0, repeat, argmax)

    def bprop_pool(self, layer, I, E, grad_I, repeat=1, relu_mask=False, argmax=None):
        """relu_mask=True also applies grad_I *= (I > 0), the mask of the ReLU layer that produced
        I, in the same pass (an extension: the reference runs it as a separate element-wise
        kernel, nervanagpu/layers.py:87-96). argmax: the record a forward pass over the same I
        left (see fprop_pool); I is then not read."""
        assert layer.sizeI == I.size
        assert layer.sizeO == E.size
        assert layer.sizeI == grad_I.size
        assert I.dtype == grad_I.dtype
        return self._execute_pool(layer, I, E, grad_I, 2 if relu_mask else 1, repeat, argmax)

    def _execute_pool(self, layer, I, O, B, mode, repeat, argmax=None):
        assert I.dtype == O.dtype
        if I.dtype.type not in (np.float16, np.float32):
            raise TypeError("pooling supports fp16 and fp32 tensors")
        desc = ctypes.byref(layer.desc)
        lib, stream, esz = self.lib, self.stream, I.dtype.itemsize
        op = {"max": 0, "avg": 1, "l2": 2}[getattr(layer, "op", "max")]
        if op != 0:
            # avg / l2: defined by the reference in numpy only (benchmarks/pool_test.py:141-146); its
            # device path runs the max kernel for them (nervanagpu/nervanagpu.py:797)
            if argmax is not None or mode == 2:
                raise ValueError("argmax records and the fused ReLU mask exist for max pooling only")
            if mode == 0:
                launch = lambda: _lib.check(lib.ng_pool_fprop_op(desc, op, esz, I.ptr, O.ptr, stream))
            else:
                launch = lambda: _lib.check(lib.ng_pool_bprop_op(desc, op, esz, I.ptr, O.ptr, B.ptr, stream))
        elif argmax is not None:
            assert argmax.nbytes >= layer.sizeO
            if mode == 0:
                launch = lambda: _lib.check(lib.ng_pool_fprop_argmax(desc, esz, I.ptr, O.ptr, argmax.ptr, stream))
            else:
                launch = lambda: _lib.check(lib.ng_pool_bprop_argmax(desc, esz, argmax.ptr, O.ptr, B.ptr,
                                                                     int(mode == 2), stream))
        elif mode == 0:
            launch = lambda: _lib.check(lib.ng_pool_fprop(desc, esz, I.ptr, O.ptr, stream))
        elif mode == 1:
            launch = lambda: _lib.check(lib.ng_pool_bprop(desc, esz, I.ptr, O.ptr, B.ptr, stream))
        else:
            launch = lambda: _lib.check(lib.ng_pool_bprop_relu(desc, esz, I.ptr, O.ptr, B.ptr, stream))
        msecs = self._timed(launch, repeat)
        if msecs is not None:
            print("%7.3f msecs (%s)" % (msecs, layer))

    # ---- GEMM ----------------------------------------------------------------------------
    @staticmethod
    def _gemm_flags(C, stochastic_round):
        rounding = C.rounding if stochastic_round is None else stochastic_round
        if rounding is True:
            rounding = 10
        return int(rounding or 0)

    def dot(self, A, B, C, alpha=1.0, beta=0.0, relu=False, repeat=1, size=None, stochastic_round=None):
        """C = alpha * A * B + beta * C, with A or B (not both) optionally a `.T` view.

        relu is applied before the beta addition. `size` selected a Maxwell tile in the reference
        and is accepted and ignored. stochastic_round: None = use C.rounding (the reference
        behaviour, nervanagpu/nervanagpu.py:1071-1072), else True / mantissa bits / 0.
        """
        assert A.dtype.type == B.dtype.type == C.dtype.type
        assert min(A.strides) == 1
        assert min(B.strides) == 1
        assert min(C.strides) == 1
        lda, ldb, ldc = max(A.strides), max(B.strides), max(C.strides)
        opA = "t" if A.is_trans else "n"
        opB = "t" if B.is_trans else "n"
        op = opA + opB
        assert op != "tt"
        m, n, k = A.shape[0], B.shape[1], A.shape[1]
        assert m == C.shape[0]
        assert n == C.shape[1]
        assert k == B.shape[0]
        if C.dtype.type is np.float32:
            raise TypeError("fp32 dot (sgemm) is not part of this library; use fp16 tensors.")
        if C.dtype.type is not np.float16:
            raise TypeError("Only floating point dot currently supported.")
        sr = self._gemm_flags(C, stochastic_round)
        lib, stream, rs = self.lib, self.stream, self.rand_state

        def launch():
            off = rs.next_offset() if sr else 0
            _lib.check(lib.ng_hgemm(A.ptr, B.ptr, C.ptr, int(A.is_trans), int(B.is_trans), m, n, k, lda, ldb, ldc,
                                    alpha, beta, int(bool(relu)), sr, rs.seed, off, stream))

        msecs = self._timed(launch, repeat)
        if msecs is not None:
            gflops = (m * n * k * 2.0) / (msecs * 1000000.0)
            print("%7.3f msecs %4.0f gflops (hgemm_%s: %d,%d,%d)" % (msecs, gflops, op, m, n, k))
            if repeat > 1:
                return gflops
        return C

    def batched_dot(self, A, B, C, alpha=1.0, beta=0.0, relu=False, repeat=1, size=None, stochastic_round=None):
        """Batched GEMM (nervanagpu/nervanagpu.py:820-957): 3-D operands carry the batch in dim 0.
        A 3-D C gives one product per batch entry; a 2-D C sums the products over the batch."""
        assert A.dtype.type == B.dtype.type == C.dtype.type
        dima = dimb = dimc = 0
        ldaz = ldbz = ldcz = 0
        batch_grid = batch_loops = 1
        if len(A.shape) == 3:
            dima, ldaz = 1, A.strides[0]
        if len(B.shape) == 3:
            dimb, ldbz = 1, B.strides[0]
        assert dima or dimb, "Tensor A or B must have 3 dims to use batched_dot"
        if len(C.shape) == 3:
            dimc, ldcz = 1, C.strides[0]
            batch_grid = C.shape[0]
            assert not dima or A.shape[0] == batch_grid
            assert not dimb or B.shape[0] == batch_grid
        elif dima:
            batch_loops = A.shape[0]
            assert not dimb or B.shape[0] == batch_loops
        elif dimb:
            batch_loops = B.shape[0]
            assert not dima or A.shape[0] == batch_loops
        m, n, k = A.shape[0 + dima], B.shape[1 + dimb], A.shape[1 + dima]
        assert m == C.shape[0 + dimc]
        assert n == C.shape[1 + dimc]
        assert k == B.shape[0 + dimb]
        lda, ldb, ldc = max(A.strides[dima:]), max(B.strides[dimb:]), max(C.strides[dimc:])
        op = ("t" if A.is_trans else "n") + ("t" if B.is_trans else "n")
        assert op != "tt"
        if C.dtype.type is not np.float16:
            raise TypeError("Only fp16 batched_dot is supported.")
        sr = self._gemm_flags(C, stochastic_round)
        lib, stream, rs = self.lib, self.stream, self.rand_state

        def launch():
            off = rs.next_offset() if sr else 0
            _lib.check(lib.ng_hgemm_batched(A.ptr, B.ptr, C.ptr, int(A.is_trans), int(B.is_trans), m, n, k,
                                            lda, ldb, ldc, alpha, beta, int(bool(relu)), sr, rs.seed, off,
                                            batch_grid, batch_loops, ldaz, ldbz, ldcz, stream))

        msecs = self._timed(launch, repeat)
        if msecs is not None:
            gflops = (batch_loops * batch_grid * m * n * k * 2.0) / (msecs * 1000000.0)
            print("%7.3f msecs %4.0f gflops (hgemm_%s: %d,%d,%d) grid:%d loops:%d" %
                  (msecs, gflops, op, m, n, k, batch_grid, batch_loops))
            if repeat > 1:
                return gflops
        return C

    def compensated_sum(self, sum_tensor, cmp_tensor, add_tensor, cmp_scale=1.0, add_scale=1.0):
        """Kahan-compensated sum += add * add_scale in the storage type
        (nervanagpu/nervanagpu.py:1107-1126, nervanagpu/float_ew.py:1430-1482)."""
        if cmp_tensor.kahan_reset and cmp_tensor.kahan_count > cmp_tensor.kahan_reset:
            cmp_scale = 0
            cmp_tensor.kahan_count = 0
        assert sum_tensor.dtype.type == cmp_tensor.dtype.type == add_tensor.dtype.type
        cmp_tensor.kahan_count += 1
        from .float_ew import call_compensated_sum
        call_compensated_sum(self, sum_tensor, cmp_tensor, add_tensor, cmp_scale, add_scale)

    # ---- lazy numpy-style operations -------------------------------------------------------
    def add(self, a, b, out=None): return OpTreeNode.build("add", a, b, out=out)
    def subtract(self, a, b, out=None): return OpTreeNode.build("sub", a, b, out=out)
    def multiply(self, a, b, out=None): return OpTreeNode.build("mul", a, b, out=out)
    def divide(self, a, b, out=None): return OpTreeNode.build("div", a, b, out=out)
    def true_divide(self, a, b, out=None): return OpTreeNode.build("div", a, b, out=out)
    def power(self, a, b, out=None): return OpTreeNode.build("pow", a, b, out=out)
    def reciprocal(self, a, out=None): return OpTreeNode.build("div", 1, a, out=out)
    def negative(self, a, out=None): return OpTreeNode.build("neg", a, None, out=out)
    def sgn(self, a, out=None): return OpTreeNode.build("sgn", a, None, out=out)
    def absolute(self, a, out=None): return OpTreeNode.build("abs", a, None, out=out)
    def fabs(self, a, out=None): return OpTreeNode.build("abs", a, None, out=out)
    def sqrt(self, a, out=None): return OpTreeNode.build("sqrt", a, None, out=out)
    def square(self, a, out=None): return OpTreeNode.build("sqr", a, None, out=out)
    def exp(self, a, out=None): return OpTreeNode.build("exp", a, None, out=out)
    def exp2(self, a, out=None): return OpTreeNode.build("exp2", a, None, out=out)
    def log(self, a, out=None): return OpTreeNode.build("log", a, None, out=out)
    def log2(self, a, out=None): return OpTreeNode.build("log2", a, None, out=out)
    def sig(self, a, out=None): return OpTreeNode.build("sig", a, None, out=out)
    def sig2(self, a, out=None): return OpTreeNode.build("sig2", a, None, out=out)
    def tanh(self, a, out=None): return OpTreeNode.build("tanh", a, None, out=out)
    def tanh2(self, a, out=None): return OpTreeNode.build("tanh2", a, None, out=out)
    def finite(self, a, out=None): return OpTreeNode.build("finite", a, None, out=out)
    def equal(self, a, b, out=None): return OpTreeNode.build("eq", a, b, out=out)
    def not_equal(self, a, b, out=None): return OpTreeNode.build("ne", a, b, out=out)
    def less(self, a, b, out=None): return OpTreeNode.build("lt", a, b, out=out)
    def less_equal(self, a, b, out=None): return OpTreeNode.build("le", a, b, out=out)
    def greater(self, a, b, out=None): return OpTreeNode.build("gt", a, b, out=out)
    def greater_equal(self, a, b, out=None): return OpTreeNode.build("ge", a, b, out=out)
    def maximum(self, a, b, out=None): return OpTreeNode.build("maximum", a, b, out=out)
    def minimum(self, a, b, out=None): return OpTreeNode.build("minimum", a, b, out=out)

    def clip(self, a, a_min, a_max, out=None):
        return self.minimum(self.maximum(a, a_min), a_max, out=out)

    def sum(self, a, axis=None, partial=None, out=None, keepdims=True):
        if axis is None:
            assert partial is not None
            return self.sum(self.sum(a, axis=1, out=partial), axis=0, out=out)
        return OpTreeNode.build("sum", a, None, axis=axis, out=out)

    def max(self, a, axis=None, partial=None, out=None, keepdims=True):
        if axis is None:
            assert partial is not None
            return self.max(self.max(a, axis=1, out=partial), axis=0, out=out)
        return OpTreeNode.build("max", a, None, axis=axis, out=out)

    def min(self, a, axis=None, partial=None, out=None, keepdims=True):
        if axis is None:
            assert partial is not None
            return self.min(self.min(a, axis=1, out=partial), axis=0, out=out)
        return OpTreeNode.build("min", a, None, axis=axis, out=out)

    def argmax(self, a, axis=1, out=None, keepdims=True):
        return OpTreeNode.build("argmax", a, None, axis=axis, out=out)

    def argmin(self, a, axis=1, out=None, keepdims=True):
        return OpTreeNode.build("argmin", a, None, axis=axis, out=out)

    def mean(self, a, axis=None, partial=None, out=None, keepdims=True):
        shape = OpTreeNode.shape(a)
        if axis is None:
            assert partial is not None
            return self.multiply(self.sum(self.sum(a, axis=1, out=partial), axis=0),
                                 1.0 / (shape[0] * shape[1]), out=out)
        return self.multiply(self.sum(a, axis=axis), 1.0 / shape[axis], out=out)

    def var(self, a, axis=None, partial=None, out=None, keepdims=True):
        if axis is None:
            assert partial is not None
            return self.mean(self.square(a - self.mean(a, axis=axis, partial=partial, out=partial[0:1, 0:1])),
                             axis=axis, partial=partial, out=out)
        return self.mean(self.square(a - self.mean(a, axis=axis)), axis=axis, out=out)

    def std(self, a, axis=None, partial=None, out=None, keepdims=True):
        return self.sqrt(self.var(a, axis=axis, partial=partial, out=out))

    def rand(self, out=None):
        return OpTreeNode.build("rand", None, None, out=out)

    def dropout(self, keep=0.5, out=None):
        return self.less_equal(self.rand(), keep, out=out)

    def take(self, a, indices, axis, out=None):
        return a.take(indices, axis, out)

    def onehot(self, indices, axis, out=None):
        if axis not in (0, 1):
            raise ValueError("bad axis for onehot")
        return OpTreeNode.build("onehot", None, None, idx=indices, axis=axis, out=out)


class OpTreeNode(tuple):
    """Node of a lazily evaluated expression: (op_dict, left, right)."""

    def __new__(cls, *args):
        return tuple.__new__(cls, args)

    # nodes hold dicts, so hash by identity
    def __hash__(self):
        return id(self)

    @staticmethod
    def build(op, a, b, out=None, **kwargs):
        for arg in (a, b):
            if not isinstance(arg, (int, float, GPUTensor, OpTreeNode, type(None))):
                return NotImplemented
        op_dict = {"op": op}
        op_dict.update(kwargs)
        node = OpTreeNode(op_dict, a, b)
        if op == "assign":
            return node.execute()
        if out is not None:
            return OpTreeNode({"op": "assign"}, out, node).execute()
        return node

    def execute(self):
        stack = self.traverse(list())
        backend = None
        for item in stack:
            if isinstance(item, GPUTensor):
                backend = item.backend
                break
        return call_compound_kernel(backend.rand_state, *stack)

    def traverse(self, stack):
        """Post-order walk producing the postfix stack."""
        for child in (self[1], self[2]):
            if type(child) is OpTreeNode:
                child.traverse(stack)
            elif child is not None:
                stack.append(child)
        stack.append(self[0])
        return stack

    @staticmethod
    def shape(node):
        if type(node) is GPUTensor:
            return node.shape
        if type(node) is OpTreeNode:
            max_shape = [1, 1]
            for item in node.traverse(list()):
                if type(item) is GPUTensor:
                    for i in range(2):
                        max_shape[i] = max(max_shape[i], item.shape[i])
            return tuple(max_shape)
        return (1, 1)

    def __add__(self, other): return self.build("add", self, other)
    def __sub__(self, other): return self.build("sub", self, other)
    def __mul__(self, other): return self.build("mul", self, other)
    def __div__(self, other): return self.build("div", self, other)
    def __truediv__(self, other): return self.build("div", self, other)
    def __pow__(self, other): return self.build("pow", self, other)
    def __radd__(self, other): return self.build("add", other, self)
    def __rsub__(self, other): return self.build("sub", other, self)
    def __rmul__(self, other): return self.build("mul", other, self)
    def __rdiv__(self, other): return self.build("div", other, self)
    def __rtruediv__(self, other): return self.build("div", other, self)
    def __rpow__(self, other): return self.build("pow", other, self)
    def __eq__(self, other): return self.build("eq", self, other)
    def __ne__(self, other): return self.build("ne", self, other)
    def __lt__(self, other): return self.build("lt", self, other)
    def __le__(self, other): return self.build("le", self, other)
    def __gt__(self, other): return self.build("gt", self, other)
    def __ge__(self, other): return self.build("ge", self, other)
    def __abs__(self): return self.build("abs", self, None)
    def __neg__(self): return self.build("neg", self, None)
