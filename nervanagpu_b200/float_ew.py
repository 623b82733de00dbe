"""Lazy element-wise / broadcast / reduction compiler.

`call_compound_kernel(rand_state, *postfix_stack)` takes the postfix stack that OpTreeNode.traverse
produces (tensors, python scalars and {"op": ...} dicts, output tensor first, "assign" last), builds
an expression graph, generates ONE CUDA kernel for it, compiles it with NVRTC through the C ABI
(memoised per expression signature) and launches it. It covers what the reference's
nervanagpu/float_ew.py:1058-1322 (call_compound_kernel) and :714-1035 (_get_compound_kernel)
cover: fused element-wise math over f16/f32/i8/u8/i16/u16/i32/u32 tensors, broadcasting along
either axis, transposed and strided views, take / onehot, reductions along axis 0 or 1
(sum, max, min, argmax, argmin) with element-wise work before, between and after them, common
sub-expression sharing (the two mean(A, axis=1) of a batch-norm expression become one
reduction), round-to-nearest, integer saturation and stochastic rounding on the store.

Code generation differs from the reference by design:
  * plain element-wise expressions over contiguous tensors run as a flat grid-stride kernel
    that moves 8 elements per thread with 16-byte accesses;
  * 2-D expressions give each row (column, for axis-0 reductions) to one warp, or to one CTA
    for long rows; reductions use warp shuffles (+ one shared-memory step per CTA);
  * random numbers come from Philox4x32-10 keyed by (seed, launch offset) and indexed by the
    element, so a rerun with the same seed repeats bit for bit.
Math is IEEE fp32 (no --use_fast_math) so that results match the numpy fp32 oracle to rounding.
"""
import ctypes
import hashlib

import numpy as np

from . import _lib

# ---------------------------------------------------------------------------------------------
# operator tables: name -> (arity, C expression template)
# ---------------------------------------------------------------------------------------------
_float_ops = {
    "assign": (2, None),
    "add": (2, "({0} + {1})"),
    "sub": (2, "({0} - {1})"),
    "mul": (2, "({0} * {1})"),
    "div": (2, "({0} / {1})"),
    "eq": (2, "(({0} == {1}) ? 1.0f : 0.0f)"),
    "ne": (2, "(({0} != {1}) ? 1.0f : 0.0f)"),
    "lt": (2, "(({0} < {1}) ? 1.0f : 0.0f)"),
    "le": (2, "(({0} <= {1}) ? 1.0f : 0.0f)"),
    "gt": (2, "(({0} > {1}) ? 1.0f : 0.0f)"),
    "ge": (2, "(({0} >= {1}) ? 1.0f : 0.0f)"),
    "minimum": (2, "fminf({0}, {1})"),
    "maximum": (2, "fmaxf({0}, {1})"),
    "pow": (2, "powf({0}, {1})"),
    "finite": (1, "(isfinite({0}) ? 1.0f : 0.0f)"),
    "neg": (1, "(-{0})"),
    "abs": (1, "fabsf({0})"),
    "sgn": (1, "copysignf(1.0f, {0})"),
    "sqrt": (1, "sqrtf({0})"),
    "sqr": (1, "({0} * {0})"),
    "exp": (1, "expf({0})"),
    "log": (1, "logf({0})"),
    "exp2": (1, "exp2f({0})"),
    "log2": (1, "log2f({0})"),
    "sig": (1, "(1.0f / (1.0f + expf(-{0})))"),
    "sig2": (1, "(1.0f / (1.0f + exp2f(-{0})))"),
    "tanh": (1, "tanhf({0})"),
    "tanh2": (1, "((exp2f(2.0f * {0}) - 1.0f) / (exp2f(2.0f * {0}) + 1.0f))"),
    "rand": (0, None),
    "onehot": (0, None),
}

_reduction_ops = ("sum", "max", "min", "argmax", "argmin")

_CTYPES = {
    "f2": "__half", "f4": "float", "u1": "unsigned char", "i1": "signed char",
    "u2": "unsigned short", "i2": "short", "u4": "unsigned int", "i4": "int",
}

_PREAMBLE = r"""
#include <cuda_fp16.h>
typedef unsigned int u32;
typedef unsigned long long u64;

struct Philox4 { u32 v[4]; };
__device__ __forceinline__ Philox4 philox(u32 c0, u32 c1, u32 c2, u32 c3, u32 k0, u32 k1) {
  #pragma unroll
  for (int r = 0; r < 10; ++r) {
    const u64 p0 = (u64)0xD2511F53u * c0, p1 = (u64)0xCD9E8D57u * c2;
    const u32 n0 = (u32)(p1 >> 32) ^ c1 ^ k0, n2 = (u32)(p0 >> 32) ^ c3 ^ k1;
    c1 = (u32)p1; c3 = (u32)p0; c0 = n0; c2 = n2;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  Philox4 o; o.v[0] = c0; o.v[1] = c1; o.v[2] = c2; o.v[3] = c3; return o;
}
struct Rng { u32 k0, k1, off; };
// 32 random bits for element `idx` of stream `stream` (0 = rounding, 16+ = rand() ops)
__device__ __forceinline__ u32 rng_u32(const Rng& g, u64 idx, u32 stream) {
  const Philox4 p = philox((u32)(idx >> 2), (u32)(idx >> 34), g.off, stream, g.k0, g.k1);
  return p.v[idx & 3];
}
__device__ __forceinline__ float rng_uniform(const Rng& g, u64 idx, u32 stream) {
  return (float)(rng_u32(g, idx, stream) >> 8) * (1.0f / 16777216.0f);
}

// stochastic rounding: add a uniform integer below one target ulp to the magnitude bits,
// then truncate toward zero (result is one of the two neighbours of x)
__device__ __forceinline__ float sr_f32(float x, u32 rnd, int mbits) {
  u32 b = __float_as_uint(x);
  if (((b >> 23) & 0xffu) == 0xffu) return x;
  const u32 mask = (1u << (23 - mbits)) - 1u;
  b += rnd & mask; b &= ~mask;
  return __uint_as_float(b);
}
__device__ __forceinline__ __half sr_f16(float x, u32 rnd, int mbits) {
  const u32 e = (__float_as_uint(x) >> 23) & 0xffu;
  if (e == 0xffu) return __float2half_rn(x);
  if (e >= 113u) return __float2half_rz(sr_f32(x, rnd, mbits));
  const float ulp = __uint_as_float((103u + (u32)(10 - mbits)) << 23);
  const float mag = fabsf(x) + (float)(rnd & 0xfffu) * (1.0f / 4096.0f) * ulp;
  return __float2half_rz(copysignf(floorf(mag / ulp) * ulp, x));
}

template <typename T> struct IO;
template <> struct IO<__half> {
  static __device__ __forceinline__ float ld(const __half* p) { return __half2float(*p); }
  static __device__ __forceinline__ void st(__half* p, float v, u32 rnd, int sr) { *p = sr ? sr_f16(v, rnd, sr) : __float2half_rn(v); }
  static __device__ __forceinline__ void ld8(const __half* p, float (&v)[8]) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&r);
    #pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); v[2*i] = f.x; v[2*i+1] = f.y; }
  }
  static __device__ __forceinline__ void st8(__half* p, const float (&v)[8], const u32 (&rnd)[8], int sr) {
    uint4 r; __half* h = reinterpret_cast<__half*>(&r);
    #pragma unroll
    for (int i = 0; i < 8; ++i) h[i] = sr ? sr_f16(v[i], rnd[i], sr) : __float2half_rn(v[i]);
    *reinterpret_cast<uint4*>(p) = r;
  }
};
template <> struct IO<float> {
  static __device__ __forceinline__ float ld(const float* p) { return *p; }
  static __device__ __forceinline__ void st(float* p, float v, u32 rnd, int sr) { *p = sr ? sr_f32(v, rnd, sr) : v; }
  static __device__ __forceinline__ void ld8(const float* p, float (&v)[8]) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    v[0]=a.x; v[1]=a.y; v[2]=a.z; v[3]=a.w; v[4]=b.x; v[5]=b.y; v[6]=b.z; v[7]=b.w;
  }
  static __device__ __forceinline__ void st8(float* p, const float (&v)[8], const u32 (&rnd)[8], int sr) {
    float o[8];
    #pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = sr ? sr_f32(v[i], rnd[i], sr) : v[i];
    reinterpret_cast<float4*>(p)[0] = make_float4(o[0], o[1], o[2], o[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(o[4], o[5], o[6], o[7]);
  }
};
// integers: round to nearest even and saturate (cvt.rni.sat)
__device__ __forceinline__ float sat_rn(float v, float lo, float hi) { return fminf(fmaxf(rintf(v), lo), hi); }
#define NG_INT_IO(T, LO, HI, CVT)                                                                   \
template <> struct IO<T> {                                                                         \
  static __device__ __forceinline__ float ld(const T* p) { return (float)(*p); }                   \
  static __device__ __forceinline__ void st(T* p, float v, u32, int) { *p = CVT; }                 \
  static __device__ __forceinline__ void ld8(const T* p, float (&v)[8]) {                          \
    T t[8];                                                                                        \
    if (sizeof(T) == 1) *reinterpret_cast<uint2*>(t) = *reinterpret_cast<const uint2*>(p);         \
    else if (sizeof(T) == 2) *reinterpret_cast<uint4*>(t) = *reinterpret_cast<const uint4*>(p);    \
    else { reinterpret_cast<uint4*>(t)[0] = reinterpret_cast<const uint4*>(p)[0];                  \
           reinterpret_cast<uint4*>(t)[1] = reinterpret_cast<const uint4*>(p)[1]; }                \
    _Pragma("unroll") for (int i = 0; i < 8; ++i) v[i] = (float)t[i];                              \
  }                                                                                                \
  static __device__ __forceinline__ void st8(T* p, const float (&vv)[8], const u32 (&)[8], int) {  \
    T t[8];                                                                                        \
    _Pragma("unroll") for (int i = 0; i < 8; ++i) { const float v = vv[i]; t[i] = CVT; }           \
    if (sizeof(T) == 1) *reinterpret_cast<uint2*>(p) = *reinterpret_cast<const uint2*>(t);         \
    else if (sizeof(T) == 2) *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(t);    \
    else { reinterpret_cast<uint4*>(p)[0] = reinterpret_cast<const uint4*>(t)[0];                  \
           reinterpret_cast<uint4*>(p)[1] = reinterpret_cast<const uint4*>(t)[1]; }                \
  }                                                                                                \
};
NG_INT_IO(unsigned char, 0.0f, 255.0f, (unsigned char)sat_rn(v, 0.0f, 255.0f))
NG_INT_IO(signed char, -128.0f, 127.0f, (signed char)sat_rn(v, -128.0f, 127.0f))
NG_INT_IO(unsigned short, 0.0f, 65535.0f, (unsigned short)sat_rn(v, 0.0f, 65535.0f))
NG_INT_IO(short, -32768.0f, 32767.0f, (short)sat_rn(v, -32768.0f, 32767.0f))
NG_INT_IO(unsigned int, 0.0f, 0.0f, __float2uint_rn(v))
NG_INT_IO(int, 0.0f, 0.0f, __float2int_rn(v))

// reductions over the THREADS threads that share a row
#define FULL 0xffffffffu
struct ArgVal { float v; int i; };
__device__ __forceinline__ float warp_sum(float v) { for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(FULL, v, o); return v; }
__device__ __forceinline__ float warp_max(float v) { for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(FULL, v, o)); return v; }
__device__ __forceinline__ float warp_min(float v) { for (int o = 16; o; o >>= 1) v = fminf(v, __shfl_xor_sync(FULL, v, o)); return v; }
// ties go to the lowest index; i < 0 marks "no element seen"
__device__ __forceinline__ ArgVal arg_better(ArgVal a, ArgVal b, bool want_max) {
  if (b.i < 0) return a;
  if (a.i < 0) return b;
  const bool b_wins = want_max ? (b.v > a.v) : (b.v < a.v);
  if (b_wins || (b.v == a.v && b.i < a.i)) return b;
  return a;
}
__device__ __forceinline__ ArgVal warp_arg(ArgVal a, bool want_max) {
  for (int o = 16; o; o >>= 1) {
    ArgVal b; b.v = __shfl_xor_sync(FULL, a.v, o); b.i = __shfl_xor_sync(FULL, a.i, o);
    a = arg_better(a, b, want_max);
  }
  return a;
}
template <int THREADS> __device__ __forceinline__ float row_reduce(float v, int kind, float* smem) {
  v = kind == 0 ? warp_sum(v) : (kind == 1 ? warp_max(v) : warp_min(v));
  if (THREADS > 32) {
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    __syncthreads();
    if (l == 0) smem[w] = v;
    __syncthreads();
    const float ident = kind == 0 ? 0.0f : (kind == 1 ? -3.402823466e+38f : 3.402823466e+38f);
    v = l < THREADS / 32 ? smem[l] : ident;
    v = kind == 0 ? warp_sum(v) : (kind == 1 ? warp_max(v) : warp_min(v));
  }
  return v;
}
template <int THREADS> __device__ __forceinline__ ArgVal row_reduce_arg(ArgVal a, bool want_max, float* smem) {
  a = warp_arg(a, want_max);
  if (THREADS > 32) {
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    __syncthreads();
    if (l == 0) { smem[w] = a.v; reinterpret_cast<int*>(smem)[32 + w] = a.i; }
    __syncthreads();
    ArgVal b; b.v = 0.0f; b.i = -1;
    if (l < THREADS / 32) { b.v = smem[l]; b.i = reinterpret_cast<int*>(smem)[32 + l]; }
    a = warp_arg(b, want_max);
  }
  return a;
}
"""


# ---------------------------------------------------------------------------------------------
# expression graph
# ---------------------------------------------------------------------------------------------
class _Node(object):
    __slots__ = ("kind", "name", "children", "slot", "extra", "key", "depth", "scalar")

    def __init__(self, kind, name=None, children=(), slot=None, extra=None):
        self.kind = kind          # "tensor" | "const" | "op" | "red" | "rand" | "onehot"
        self.name = name
        self.children = tuple(children)
        self.slot = slot
        self.extra = extra
        ck = tuple(c.key for c in self.children)
        self.key = (kind, name, slot, extra, ck)
        if kind == "red":
            self.depth = 1 + self.children[0].depth
        else:
            self.depth = max([c.depth for c in self.children] + [0])
        if kind in ("const", "red"):
            self.scalar = True
        elif kind == "op":
            self.scalar = all(c.scalar for c in self.children)
        else:
            self.scalar = False


class _Plan(object):
    """Everything derived from one postfix stack: graph, kernel key, arguments, launch shape."""


def _is_2d_special(t):
    return len(t.shape) < 2 or (len(t.shape) == 2 and (t.shape[0] == 1 or t.shape[1] == 1))


def _analyse(args):
    """Build the expression graph and the argument list from a postfix stack."""
    from .nervanagpu import GPUTensor  # local import: nervanagpu imports this module

    plan = _Plan()
    out = None
    axis = 1
    reduction = broadcast = transpose = takeop = False
    contiguous = True
    size = None
    same_size = True
    shape0 = None
    same_shape = True
    for arg in args:
        if type(arg) is dict:
            op_name = arg["op"]
            if op_name in _reduction_ops:
                if arg.get("axis", None) not in (0, 1):
                    raise ValueError("Only reduction along an axis currently supported")
                if reduction and arg["axis"] != axis:
                    raise ValueError("Reduction only allowed along one axis per kernel.")
                reduction = True
                axis = arg["axis"]
            elif op_name == "onehot":
                takeop = True
        elif isinstance(arg, GPUTensor):
            if out is None:
                out = arg
            if arg.is_trans and len(arg.shape) > 1 and min(arg.shape) > 1:
                transpose = True
            elif arg.take_array:
                takeop = True
            elif _is_2d_special(arg):
                broadcast = True
            elif not arg.is_contiguous:
                contiguous = False
            if not arg.is_contiguous:
                contiguous = False
            if size is None:
                size, shape0 = arg.size, tuple(arg.shape)
            else:
                same_size = same_size and arg.size == size
                same_shape = same_shape and tuple(arg.shape) == shape0
    if out is None:
        raise TypeError("the first operand of an assignment must be a GPUTensor")
    # Vectors and single rows/columns only broadcast when they meet a tensor of another shape;
    # operands that all share one shape (any rank) are walked in memory order.
    if same_shape:
        broadcast = False
    flat = not (broadcast or reduction or transpose or takeop) and contiguous and same_size

    tensors = []       # slot -> dict(tensor, shape, strides, take)
    slot_of = {}       # id(tensor) -> slot
    consts = []        # slot -> float
    const_slot = {}
    red_lengths = []   # per reduction node: axis length of its input
    nodes = {}         # key -> node (common sub-expression sharing)
    rand_serial = [0]

    def intern(node):
        return nodes.setdefault(node.key, node)

    stack = []         # (node, shape)
    result = None
    for arg in args:
        if isinstance(arg, GPUTensor):
            if flat:
                shape = (1, arg.size)
            else:
                if len(arg.shape) != 2:
                    raise ValueError("Operations that are not simple elementwise are only currently "
                                     "supported in 2 dimensions.")
                shape = tuple(arg.shape)
            if id(arg) in slot_of:
                slot = slot_of[id(arg)]
            else:
                slot = len(tensors)
                slot_of[id(arg)] = slot
                entry = {"tensor": arg, "dtype": arg.dtype.str[1:], "take": 0, "take_ptr": None}
                if flat:
                    entry["strides"] = (0, 1)
                else:
                    s = list(arg.strides)
                    if arg.shape[0] == 1:
                        s[0] = 0
                    if arg.shape[1] == 1:
                        s[1] = 0
                    if axis == 0:
                        s = s[::-1]
                    entry["strides"] = tuple(s)
                    if arg.take_array:
                        idx_tensor, take_axis = arg.take_array
                        # 1 = index the kernel's row coordinate, 2 = its column coordinate
                        kernel_axis = take_axis if axis == 1 else 1 - take_axis
                        entry["take"] = 1 + kernel_axis
                        entry["take_ptr"] = idx_tensor
                tensors.append(entry)
            stack.append((intern(_Node("tensor", slot=slot)), shape))

        elif type(arg) in (int, float) or isinstance(arg, (np.integer, np.floating)):
            val = float(arg)
            if val not in const_slot:
                const_slot[val] = len(consts)
                consts.append(val)
            stack.append((intern(_Node("const", slot=const_slot[val])), (1, 1)))

        elif type(arg) is dict:
            op_name = arg["op"]
            if op_name in _float_ops:
                arity = _float_ops[op_name][0]
                operands = [stack.pop() for _ in range(arity)][::-1]
                max_shape = [1, 1]
                for _, shape in operands:
                    for i in range(2):
                        if shape[i] != max_shape[i]:
                            if shape[i] == 1 or max_shape[i] == 1:
                                max_shape[i] = max(max_shape[i], shape[i])
                            else:
                                raise TypeError("Input shape:%s not compatible" % (shape,))
                if op_name == "assign":
                    result = (operands[0][0], operands[1][0], tuple(max_shape))
                elif op_name == "rand":
                    rand_serial[0] += 1
                    stack.append((_Node("rand", extra=rand_serial[0]), (1, 1)))
                elif op_name == "onehot":
                    idx_tensor = arg["idx"]
                    hot_axis = arg["axis"] if axis == 1 else 1 - arg["axis"]
                    if id(idx_tensor) in slot_of:
                        slot = slot_of[id(idx_tensor)]
                    else:
                        slot = len(tensors)
                        slot_of[id(idx_tensor)] = slot
                        tensors.append({"tensor": idx_tensor, "dtype": idx_tensor.dtype.str[1:], "take": 0,
                                        "take_ptr": None, "strides": (0, 0), "raw_index": True})
                    stack.append((intern(_Node("onehot", slot=slot, extra=hot_axis)), (1, 1)))
                else:
                    stack.append((intern(_Node("op", op_name, [o[0] for o in operands])), tuple(max_shape)))
            elif op_name in _reduction_ops:
                node, shape = stack.pop()
                shape = list(shape)
                red = intern(_Node("red", op_name, [node]))
                if not hasattr(plan, "_red_len"):
                    plan._red_len = {}
                plan._red_len.setdefault(red.key, shape[axis] if not flat else shape[1])
                shape[axis] = 1
                stack.append((red, tuple(shape)))
            else:
                raise TypeError("%s is not a valid operation" % op_name)
        else:
            raise TypeError("args must be instance of GPUTensor, int, float, or dict (for operators)")

    if result is None:
        raise TypeError("expression does not end in an assignment")
    out_node, value_node, max_shape = result
    if out_node.kind != "tensor" or out_node.slot != 0:
        raise TypeError("the assignment target must be the first tensor of the expression")

    plan.out = out
    plan.flat = flat
    plan.axis = axis
    plan.tensors = tensors
    plan.consts = consts
    plan.value = value_node
    plan.max_shape = max_shape
    plan.red_len = getattr(plan, "_red_len", {})
    return plan


# ---------------------------------------------------------------------------------------------
# code generation
# ---------------------------------------------------------------------------------------------
class _Emitter(object):
    """Emits C statements for graph nodes. Row-scope values (constants, reduction results and
    anything computed only from those) are emitted once per row; everything else per element."""

    def __init__(self, plan, vec):
        self.plan = plan
        self.vec = vec
        self.row_names = {}
        self.row_lines = []
        self.counter = 0
        self.red_names = {}

    def fresh(self, prefix="v"):
        self.counter += 1
        return "%s%d" % (prefix, self.counter)

    def load_expr(self, slot):
        t = self.plan.tensors[slot]
        if self.plan.flat:
            return "a%d[j]" % slot if self.vec else "IO<%s>::ld(p%d + idx)" % (_CTYPES[t["dtype"]], slot)
        if isinstance(self.vec, tuple):          # row-vector mode: values are already in registers
            return "a%d[ch][j]" % slot if self.vec[4][slot] == "v" else "b%d" % slot
        row = "row" if t["take"] != 1 else "take%d[row]" % slot
        col = "col" if t["take"] != 2 else "take%d[col]" % slot
        return "IO<%s>::ld(p%d + (long long)(%s) * s%d_0 + (long long)(%s) * s%d_1)" % (
            _CTYPES[t["dtype"]], slot, row, slot, col, slot)

    def emit(self, node, loop_names, loop_lines):
        """Returns the C name holding `node`; appends any statements needed to define it."""
        if node.scalar:
            return self.emit_row(node)
        if node.key in loop_names:
            return loop_names[node.key]
        if node.kind == "tensor":
            expr = self.load_expr(node.slot)
        elif node.kind == "rand":
            expr = "rng_uniform(rng, (u64)lin, %du)" % (16 + node.extra)
        elif node.kind == "onehot":
            t = self.plan.tensors[node.slot]
            # hot axis 0: value(row, col) = idx[col] == row ; hot axis 1: idx[row] == col
            if node.extra == 0:
                expr = "((int)p%d[col] == row ? 1.0f : 0.0f)" % node.slot
            else:
                expr = "((int)p%d[row] == col ? 1.0f : 0.0f)" % node.slot
        elif (node.name == "div" and len(node.children) == 2 and node.children[1].scalar
              and not node.children[0].scalar):
            # x / s with s fixed for the whole row (a reduction result, a constant): the reciprocal
            # is taken once per row and every element multiplies by it. An IEEE division per
            # element made the batch-norm kernel issue-bound; the product differs from the
            # quotient by at most one fp32 ulp.
            num = self.emit(node.children[0], loop_names, loop_lines)
            den = self.emit_row(node.children[1])
            inv_key = ("recip", node.children[1].key)
            if inv_key not in self.row_names:
                inv = self.fresh("s")
                self.row_lines.append("const float %s = 1.0f / %s;" % (inv, den))
                self.row_names[inv_key] = inv
            expr = "(%s * %s)" % (num, self.row_names[inv_key])
        else:
            names = [self.emit(c, loop_names, loop_lines) for c in node.children]
            expr = _float_ops[node.name][1].format(*names)
        name = self.fresh()
        loop_lines.append("const float %s = %s;" % (name, expr))
        loop_names[node.key] = name
        return name

    def emit_row(self, node):
        if node.key in self.row_names:
            return self.row_names[node.key]
        if node.kind == "const":
            name = "c%d" % node.slot
        elif node.kind == "red":
            name = self.red_names[node.key]   # defined by the stage that computed it
        else:
            names = [self.emit_row(c) for c in node.children]
            name = self.fresh("s")
            self.row_lines.append("const float %s = %s;" % (name, _float_ops[node.name][1].format(*names)))
        self.row_names[node.key] = name
        return name


def _collect_reductions(node, found):
    for c in node.children:
        _collect_reductions(c, found)
    if node.kind == "red" and node.key not in found:
        found[node.key] = node
    return found


_RED_INIT = {"sum": "0.0f", "max": "-3.402823466e+38f", "min": "3.402823466e+38f"}
_RED_KIND = {"sum": 0, "max": 1, "min": 2}


def _signature(plan, vec, threads, sr):
    """Hashable description of the generated code (independent of pointers and sizes)."""
    tens = tuple((t["dtype"], t["take"], bool(t.get("raw_index"))) for t in plan.tensors)
    return (plan.flat, vec, threads, bool(sr), plan.axis, tens, len(plan.consts), plan.value.key)


def _generate(plan, vec, threads, sr, kernel_name):
    em = _Emitter(plan, vec)
    out_t = plan.tensors[0]
    out_c = _CTYPES[out_t["dtype"]]
    params = []
    for i, t in enumerate(plan.tensors):
        const = "" if i == 0 else "const "
        params.append("%s%s* __restrict__ p%d" % (const, _CTYPES[t["dtype"]], i) if i else
                      "%s* p%d" % (_CTYPES[t["dtype"]], i))
        if not plan.flat:
            params.append("int s%d_0" % i)
            params.append("int s%d_1" % i)
            if t["take"]:
                params.append("const int* __restrict__ take%d" % i)
    for i in range(len(plan.consts)):
        params.append("float c%d" % i)
    reds = _collect_reductions(plan.value, {})
    red_list = sorted(reds.values(), key=lambda n: n.depth)
    for i, r in enumerate(red_list):
        params.append("int n_red%d" % i)
    params += ["long long n_rows", "int n_cols", "u32 seed_lo", "u32 seed_hi", "u32 rng_off", "int sr_bits"]

    src = [_PREAMBLE, 'extern "C" __global__ void __launch_bounds__(%d) %s(%s) {' %
           (max(threads, 32) if plan.flat else (threads if threads > 32 else 256), kernel_name, ", ".join(params)),
           "  Rng rng; rng.k0 = seed_lo; rng.k1 = seed_hi; rng.off = rng_off;"]

    if plan.flat:
        loop_names, loop_lines = {}, []
        value = em.emit(plan.value, loop_names, loop_lines)
        src += ["  " + l for l in em.row_lines]
        if vec:
            src.append("  const long long n_vec = n_rows;  // groups of 8 elements")
            src.append("  for (long long g = blockIdx.x * (long long)blockDim.x + threadIdx.x; g < n_vec; "
                       "g += (long long)gridDim.x * blockDim.x) {")
            src.append("    const long long idx = g * 8;")
            used = sorted(set(int(k[2]) for k in loop_names if k[0] == "tensor"))
            for s in used:
                src.append("    float a%d[8]; IO<%s>::ld8(p%d + idx, a%d);" %
                           (s, _CTYPES[plan.tensors[s]["dtype"]], s, s))
            src.append("    float o[8]; u32 rnd[8];")
            src.append("    #pragma unroll")
            src.append("    for (int j = 0; j < 8; ++j) {")
            src.append("      const long long lin = idx + j; (void)lin;")
            src += ["      " + l for l in loop_lines]
            src.append("      o[j] = %s;" % value)
            src.append("      rnd[j] = 0;")
            src.append("    }")
            if sr:
                src.append("    if (sr_bits) {")
                src.append("      if (sizeof(%s) == 2 && sr_bits >= 7) {" % out_c)
                src.append("        const Philox4 r = philox((u32)g, (u32)(g >> 32), rng_off, 1u, seed_lo, seed_hi);")
                src.append("        #pragma unroll")
                src.append("        for (int j = 0; j < 4; ++j) { rnd[2*j] = r.v[j] & 0xffffu; rnd[2*j+1] = r.v[j] >> 16; }")
                src.append("      } else {")
                src.append("        #pragma unroll")
                src.append("        for (int j = 0; j < 8; ++j) rnd[j] = rng_u32(rng, (u64)(idx + j), 0u);")
                src.append("      }")
                src.append("    }")
            src.append("    IO<%s>::st8(p0 + idx, o, rnd, sr_bits);" % out_c)
            src.append("  }")
        else:
            src.append("  const long long n_elem = n_rows;")
            src.append("  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < n_elem; "
                       "idx += (long long)gridDim.x * blockDim.x) {")
            src.append("    const long long lin = idx; (void)lin;")
            src += ["    " + l for l in loop_lines]
            src.append("    IO<%s>::st(p0 + idx, %s, %s, sr_bits);" %
                       (out_c, value, "sr_bits ? rng_u32(rng, (u64)idx, 0u) : 0u" if sr else "0u"))
            src.append("  }")
        src.append("}")
        return "\n".join(src)

    if isinstance(vec, tuple):
        return _generate_rowvec(plan, em, vec, sr, src, red_list, out_c)

    # ---- 2-D: one row per warp (THREADS == 32) or per CTA ---------------------------------
    if threads == 32:
        src.append("  const int tid = threadIdx.x & 31;")
        src.append("  const long long row_ll = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);")
        src.append("  if (row_ll >= n_rows) return;")
        src.append("  float* smem = nullptr;")
    else:
        src.append("  __shared__ float smem_buf[64];")
        src.append("  float* smem = smem_buf;")
        src.append("  const int tid = threadIdx.x;")
        src.append("  const long long row_ll = blockIdx.x;")
    src.append("  const int row = (int)row_ll;")
    T = "32" if threads == 32 else str(threads)

    max_depth = max([r.depth for r in red_list] + [0])
    for stage in range(1, max_depth + 1):
        stage_reds = [r for r in red_list if r.depth == stage]
        loop_names, loop_lines = {}, []
        mark = len(em.row_lines)
        updates = []
        inits = {}
        for r in stage_reds:
            i = red_list.index(r)
            arg = em.emit(r.children[0], loop_names, loop_lines)
            acc = "r%d" % i
            if r.name in ("argmax", "argmin"):
                src_init = "  ArgVal %s; %s.v = 0.0f; %s.i = -1;" % (acc, acc, acc)
                cmp_ = ">" if r.name == "argmax" else "<"
                updates.append("if (%s.i < 0 || %s %s %s.v) { %s.v = %s; %s.i = col; }" %
                               (acc, arg, cmp_, acc, acc, arg, acc))
            else:
                src_init = "  float %s = %s;" % (acc, _RED_INIT[r.name])
                if r.name == "sum":
                    updates.append("%s += %s;" % (acc, arg))
                elif r.name == "max":
                    updates.append("%s = fmaxf(%s, %s);" % (acc, acc, arg))
                else:
                    updates.append("%s = fminf(%s, %s);" % (acc, acc, arg))
            inits[r.key] = src_init
        # row-scope values this stage depends on
        src += ["  " + l for l in em.row_lines[mark:]]
        for r in stage_reds:
            src.append(inits[r.key])
        n_name = "n_red%d" % red_list.index(stage_reds[0])
        src.append("  for (int col = tid; col < %s; col += %s) {" % (n_name, T))
        src.append("    const long long lin = (long long)row * %s + col; (void)lin;" % n_name)
        src += ["    " + l for l in loop_lines]
        src += ["    " + u for u in updates]
        src.append("  }")
        for r in stage_reds:
            i = red_list.index(r)
            if r.name in ("argmax", "argmin"):
                src.append("  r%d = row_reduce_arg<%s>(r%d, %s, smem);" %
                           (i, T, i, "true" if r.name == "argmax" else "false"))
                src.append("  const float rr%d = (float)r%d.i;" % (i, i))
            else:
                src.append("  const float rr%d = row_reduce<%s>(r%d, %d, smem);" % (i, T, i, _RED_KIND[r.name]))
            em.red_names[r.key] = "rr%d" % i

    loop_names, loop_lines = {}, []
    mark = len(em.row_lines)
    value = em.emit(plan.value, loop_names, loop_lines)
    src += ["  " + l for l in em.row_lines[mark:]]
    src.append("  for (int col = tid; col < n_cols; col += %s) {" % T)
    src.append("    const long long lin = (long long)row * n_cols + col; (void)lin;")
    src += ["    " + l for l in loop_lines]
    src.append("    IO<%s>::st(p0 + (long long)row * s0_0 + (long long)col * s0_1, %s, %s, sr_bits);" %
               (out_c, value, "sr_bits ? rng_u32(rng, (u64)lin, 0u) : 0u" if sr else "0u"))
    src.append("  }")
    src.append("}")
    return "\n".join(src)


def _generate_rowvec(plan, em, cfg, sr, src, red_list, out_c):
    _, lpr, nch, cached, kinds = cfg
    src.append("  const int lane = threadIdx.x & 31, sub = lane / %d, li = lane %% %d;" % (lpr, lpr))
    src.append("  const long long row_ll = (blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5)) * %d + sub;"
               % (32 // lpr))
    src.append("  const bool row_live = row_ll < n_rows;")
    src.append("  const int row = row_live ? (int)row_ll : 0;   // idle lanes shadow row 0 so shuffles stay uniform")
    vslots = [i for i, k in enumerate(kinds) if k == "v"]

    def emit_loads(indent, ch_expr, slots):
        out = []
        for sl in slots:
            ct = _CTYPES[plan.tensors[sl]["dtype"]]
            out.append("%sIO<%s>::ld8(p%d + (long long)row * s%d_0 + col0, a%d[%s]);" % (indent, ct, sl, sl, sl, ch_expr))
        return out

    for sl, k in enumerate(kinds):
        if k == "b":
            src.append("  const float b%d = IO<%s>::ld(p%d + (long long)row * s%d_0);" %
                       (sl, _CTYPES[plan.tensors[sl]["dtype"]], sl, sl))
    arr = nch if cached else 1
    used_all = set()

    def tensors_used(node, acc):
        for c in node.children:
            tensors_used(c, acc)
        if node.kind == "tensor":
            acc.add(node.slot)
        return acc

    tensors_used(plan.value, used_all)
    in_slots = [sl for sl in vslots if sl in used_all]
    for sl in in_slots:
        src.append("  float a%d[%d][8];" % (sl, arr))
    if cached:
        src.append("  #pragma unroll")
        src.append("  for (int ch = 0; ch < %d; ++ch) {" % nch)
        src.append("    const int col0 = (ch * %d + li) * 8;" % lpr)
        src.append("    if (col0 < n_cols) {")
        src += emit_loads("      ", "ch", in_slots)
        src.append("    } else {")
        for sl in in_slots:
            src.append("      for (int j = 0; j < 8; ++j) a%d[ch][j] = 0.0f;" % sl)
        src.append("    }")
        src.append("  }")

    def chunk_loop_open():
        lines = ["  #pragma unroll" if cached else "  // rows too long for registers: re-read per stage",
                 "  for (int chi = 0; chi < %d; ++chi) {" % nch,
                 "    const int ch = %s;" % ("chi" if cached else "0"),
                 "    const int col0 = (chi * %d + li) * 8;" % lpr,
                 "    if (col0 >= n_cols) continue;"]
        if not cached:
            lines += emit_loads("    ", "0", in_slots)
        return lines

    max_depth = max([r.depth for r in red_list] + [0])
    for stage in range(1, max_depth + 1):
        stage_reds = [r for r in red_list if r.depth == stage]
        loop_names, loop_lines = {}, []
        mark = len(em.row_lines)
        updates, inits = [], []
        for r in stage_reds:
            i = red_list.index(r)
            arg = em.emit(r.children[0], loop_names, loop_lines)
            acc = "r%d" % i
            if r.name in ("argmax", "argmin"):
                inits.append("  ArgVal %s; %s.v = 0.0f; %s.i = -1;" % (acc, acc, acc))
                cmp_ = ">" if r.name == "argmax" else "<"
                updates.append("if (%s.i < 0 || %s %s %s.v) { %s.v = %s; %s.i = col; }" % (acc, arg, cmp_, acc, acc, arg, acc))
            else:
                inits.append("  float %s = %s;" % (acc, _RED_INIT[r.name]))
                updates.append({"sum": "%s += %s;", "max": "%s = fmaxf(%s, %s);", "min": "%s = fminf(%s, %s);"}[r.name] %
                               ((acc, arg) if r.name == "sum" else (acc, acc, arg)))
        src += ["  " + l for l in em.row_lines[mark:]]
        src += inits
        src += chunk_loop_open()
        src.append("    #pragma unroll")
        src.append("    for (int j = 0; j < 8; ++j) {")
        src.append("      const int col = col0 + j; const long long lin = (long long)row * n_cols + col; (void)lin; (void)col;")
        src += ["      " + l for l in loop_lines]
        src += ["      " + u for u in updates]
        src.append("    }")
        src.append("  }")
        for r in stage_reds:
            i = red_list.index(r)
            if r.name in ("argmax", "argmin"):
                want = "true" if r.name == "argmax" else "false"
                src.append("  for (int o = %d; o; o >>= 1) { ArgVal t_; t_.v = __shfl_xor_sync(FULL, r%d.v, o); "
                           "t_.i = __shfl_xor_sync(FULL, r%d.i, o); r%d = arg_better(r%d, t_, %s); }" %
                           (lpr // 2, i, i, i, i, want))
                src.append("  const float rr%d = (float)r%d.i;" % (i, i))
            else:
                op = {"sum": "r%d += t_;", "max": "r%d = fmaxf(r%d, t_);", "min": "r%d = fminf(r%d, t_);"}[r.name]
                op = op % ((i,) if r.name == "sum" else (i, i))
                src.append("  for (int o = %d; o; o >>= 1) { const float t_ = __shfl_xor_sync(FULL, r%d, o); %s }" %
                           (lpr // 2, i, op))
                src.append("  const float rr%d = r%d;" % (i, i))
            em.red_names[r.key] = "rr%d" % i

    loop_names, loop_lines = {}, []
    mark = len(em.row_lines)
    value = em.emit(plan.value, loop_names, loop_lines)
    src += ["  " + l for l in em.row_lines[mark:]]
    src += chunk_loop_open()
    src.append("    float o[8]; u32 rnd[8];")
    src.append("    #pragma unroll")
    src.append("    for (int j = 0; j < 8; ++j) {")
    src.append("      const int col = col0 + j; const long long lin = (long long)row * n_cols + col; (void)lin; (void)col;")
    src += ["      " + l for l in loop_lines]
    src.append("      o[j] = %s;" % value)
    src.append("      rnd[j] = %s;" % ("sr_bits ? rng_u32(rng, (u64)lin, 0u) : 0u" if sr else "0u"))
    src.append("    }")
    src.append("    if (row_live) IO<%s>::st8(p0 + (long long)row * s0_0 + col0, o, rnd, sr_bits);" % out_c)
    src.append("  }")
    src.append("}")
    return "\n".join(src)


# ---------------------------------------------------------------------------------------------
# compile cache and launch
# ---------------------------------------------------------------------------------------------
_kernel_cache = {}
_last_source = [None]


def _get_kernel(plan, vec, threads, sr):
    sig = _signature(plan, vec, threads, sr)
    hit = _kernel_cache.get(sig)
    if hit is not None:
        return hit
    name = "ew_" + hashlib.sha1(repr(sig).encode()).hexdigest()[:16]
    source = _generate(plan, vec, threads, sr, name)
    _last_source[0] = source
    lib = _lib.init()
    handle = ctypes.c_void_p()
    rc = lib.ng_ew_compile(source.encode(), name.encode(), 0, ctypes.byref(handle))
    if rc != 0:
        log = lib.ng_ew_compile_log().decode("utf-8", "replace")
        raise _lib.NervanaError(rc, lib.ng_last_error().decode("utf-8", "replace") + "\n" + log)
    _kernel_cache[sig] = handle
    return handle


def generate_source(*args):
    """Source text of the kernel that call_compound_kernel would run for this postfix stack
    (no device needed). Returns (source, launch description)."""
    plan = _analyse(args)
    vec, threads, sr = _launch_shape(plan)
    return _generate(plan, vec, threads, sr, "ew_preview"), {"flat": plan.flat, "vec": vec, "threads": threads}


def _round_bits(out):
    rounding = out.rounding
    if not rounding or out.dtype.kind != "f":
        return 0
    if rounding is True:
        rounding = 10
    limit = 10 if out.dtype.itemsize == 2 else 15
    return max(min(int(rounding), limit), 1)


def _launch_shape(plan):
    sr = _round_bits(plan.out)
    if plan.flat:
        size = plan.out.size
        aligned = all(t["tensor"].ptr % 16 == 0 for t in plan.tensors)
        vec = size % 8 == 0 and aligned and size > 0
        return vec, 256, sr
    depth = max(list(plan.red_len.values()) + [plan.max_shape[plan.axis]])
    rowvec = _rowvec_config(plan, depth)
    if rowvec is not None:
        return rowvec, 32, sr
    if depth <= 1024:
        threads = 32
    elif depth <= 4096:
        threads = 256
    else:
        threads = 1024
    return False, threads, sr


def _rowvec_config(plan, depth):
    """Row-vector mode for 2-D expressions over short rows with unit inner stride: every lane
    holds 8 consecutive elements per 16-byte access, 32/LPR rows share a warp, each tensor is read
    from memory once and kept in registers across the reduction stages.
    Returns ("row", lanes_per_row, chunks_per_lane, cached, kinds) or None."""
    n_cols = plan.max_shape[plan.axis]
    if n_cols % 8 != 0 or n_cols > 4096 or n_cols < 8:
        return None
    if any(v != n_cols for v in plan.red_len.values()):
        return None
    kinds = []
    for i, t in enumerate(plan.tensors):
        if t["take"] or t.get("raw_index"):
            return None
        s0, s1 = t["strides"]
        item = int(t["dtype"][1:])
        if s1 == 1:
            if t["tensor"].ptr % 16 != 0 or (s0 * item) % 16 != 0:
                return None
            kinds.append("v")
        elif s1 == 0 and i != 0:
            kinds.append("b")
        else:
            return None
    chunks = n_cols // 8
    lpr = 32
    for cand in (1, 2, 4, 8, 16):
        if chunks == cand:
            lpr = cand
    ch = (chunks + lpr - 1) // lpr
    return ("row", lpr, ch, ch <= 4, "".join(kinds))


class _Launch(object):
    """A prepared launch: compiled kernel, marshalled arguments, grid. Reused while the same
    expression is applied to tensors with the same device layout (the common case in a training
    loop), so that the per-call host cost is a dictionary lookup and one C call."""
    __slots__ = ("kernel", "holders", "argv", "grid", "block", "offset_holder", "keepalive")


_launch_cache = {}
_LAUNCH_CACHE_LIMIT = 4096


def _tensor_key(t):
    take = t.take_array
    return (t.ptr, t.shape, t.strides, t.dtype.str, t.is_trans, t.rounding,
            None if not take else (take[0].ptr, take[0].shape, take[1]))


def _stack_key(args):
    key = []
    for a in args:
        if type(a) is dict:
            if "idx" in a:
                key.append(tuple(sorted((k, (_tensor_key(v) if k == "idx" else v)) for k, v in a.items())))
            else:
                key.append(tuple(sorted(a.items())))
        elif hasattr(a, "gpudata"):
            key.append(_tensor_key(a))
        else:
            key.append(("c", float(a)))
    return tuple(key)


def _prepare(args):
    plan = _analyse(args)
    out = plan.out
    vec, threads, sr = _launch_shape(plan)
    kernel = _get_kernel(plan, vec, threads, sr)
    holders = []

    def push(ctype, value):
        holders.append(ctype(value))

    for i, t in enumerate(plan.tensors):
        push(ctypes.c_void_p, t["tensor"].ptr)
        if not plan.flat:
            push(ctypes.c_int, t["strides"][0])
            push(ctypes.c_int, t["strides"][1])
            if t["take"]:
                push(ctypes.c_void_p, t["take_ptr"].ptr)
    for c in plan.consts:
        push(ctypes.c_float, c)
    reds = sorted(_collect_reductions(plan.value, {}).values(), key=lambda n: n.depth)
    for r in reds:
        push(ctypes.c_int, plan.red_len[r.key])

    sm = _lib.sm_count()
    if plan.flat:
        n = out.size // 8 if vec else out.size
        push(ctypes.c_longlong, n)
        push(ctypes.c_int, 0)
        blocks = max(1, min((n + 255) // 256, sm * 16))
        grid, block = (blocks, 1, 1), (256, 1, 1)
    else:
        axis = plan.axis
        n_rows = plan.max_shape[1 - axis]
        n_cols = plan.max_shape[axis]
        push(ctypes.c_longlong, n_rows)
        push(ctypes.c_int, n_cols)
        if isinstance(vec, tuple):
            rows_per_block = 8 * (32 // vec[1])
            grid, block = ((n_rows + rows_per_block - 1) // rows_per_block, 1, 1), (256, 1, 1)
        elif threads == 32:
            rows_per_block = 8
            grid, block = ((n_rows + rows_per_block - 1) // rows_per_block, 1, 1), (32 * rows_per_block, 1, 1)
        else:
            grid, block = (n_rows, 1, 1), (threads, 1, 1)
    launch = _Launch()
    push(ctypes.c_uint, 0)          # seed lo (filled per call)
    push(ctypes.c_uint, 0)          # seed hi
    push(ctypes.c_uint, 0)          # rng offset
    push(ctypes.c_int, sr)
    launch.kernel = kernel
    launch.holders = holders
    launch.argv = (ctypes.c_void_p * len(holders))(*[ctypes.cast(ctypes.pointer(h), ctypes.c_void_p) for h in holders])
    launch.grid, launch.block = grid, block
    # The entry holds raw addresses, not tensors: it is found again only through a key made of the
    # same addresses and layouts, so it never outlives the meaning of its arguments.
    launch.keepalive = None
    return launch


def call_compound_kernel(rand_state, *args):
    """Run the expression given as a postfix stack, e.g. for C[:] = 2.5 * A * B + 1:
    (C, 2.5, A, {"op":"mul"}, B, {"op":"mul"}, 1, {"op":"add"}, {"op":"assign"})."""
    out = None
    for a in args:
        if hasattr(a, "gpudata"):
            out = a
            break
    if out is None:
        raise TypeError("the first operand of an assignment must be a GPUTensor")
    key = _stack_key(args)
    launch = _launch_cache.get(key)
    if launch is None:
        if out.size == 0:
            _analyse(args)          # still validate the expression
            return out
        launch = _prepare(args)
        if len(_launch_cache) >= _LAUNCH_CACHE_LIMIT:
            _launch_cache.clear()
        _launch_cache[key] = launch
    h = launch.holders
    seed = rand_state.seed if rand_state is not None else 0
    h[-4].value = seed & 0xFFFFFFFF
    h[-3].value = (seed >> 32) & 0xFFFFFFFF
    h[-2].value = rand_state.next_offset() if rand_state is not None else 0
    backend = out.backend
    repeat = backend.bench if (backend is not None and type(backend.bench) is int and backend.bench > 1) else 1
    lib = _lib.init()
    g, b = launch.grid, launch.block
    for _ in range(repeat):
        _lib.check(lib.ng_ew_launch(launch.kernel, g[0], g[1], g[2], b[0], b[1], b[2], 0, launch.argv,
                                    backend.stream if backend is not None else None))
    return out


def fp32_convert(src_tensor, dest_tensor):
    """dest[:] = src (fp32 scratch -> destination dtype), nervanagpu/float_ew.py:1325-1333."""
    return call_compound_kernel(None, dest_tensor, src_tensor, {"op": "assign"})


def call_compensated_sum(backend, sum_tensor, cmp_tensor, add_tensor, cmp_scale, add_scale):
    """Kahan summation in the storage dtype (nervanagpu/float_ew.py:1430-1482):
        y = add * add_scale - cmp * cmp_scale ; t = sum + y ; cmp = (t - sum) - y ; sum = t
    with t and cmp rounded to the storage type as they are stored. Expressed with the lazy
    compiler as three fused assignments on flat views."""
    s, c, a = sum_tensor, cmp_tensor, add_tensor
    tmp = backend.empty(s.shape, dtype=s.dtype)
    y = backend.empty(s.shape, dtype=np.float32)
    y[:] = a * add_scale - c * cmp_scale
    tmp[:] = s + y
    c[:] = (tmp - s) - y
    s[:] = tmp
