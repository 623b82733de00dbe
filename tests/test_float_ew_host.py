"""Host-side tests of the lazy element-wise compiler: op-tree -> postfix stack -> generated CUDA
source, compiled for sm_100a with NVRTC (no device needed)."""
import numpy as np
import pytest

from nervanagpu_b200 import float_ew
from nervanagpu_b200.nervanagpu import NervanaGPU, OpTreeNode


@pytest.fixture()
def ops():
    # the lazy-op helpers only build trees; they need no device
    return NervanaGPU.__new__(NervanaGPU)


def _source(out, expr):
    stack = OpTreeNode({"op": "assign"}, out, expr).traverse([])
    return float_ew.generate_source(*stack)


def _compiles(lib, source):
    rc = lib.ng_ew_compile_only(source.encode(), 0)
    assert rc == 0, lib.ng_last_error().decode() + "\n" + lib.ng_ew_compile_log().decode()


def test_postfix_order(fake_tensor):
    A, B, C = fake_tensor((4, 8)), fake_tensor((4, 8)), fake_tensor((4, 8))
    stack = OpTreeNode({"op": "assign"}, C, 2.5 * A * B + 1).traverse([])
    kinds = [x["op"] if isinstance(x, dict) else ("T" if hasattr(x, "shape") else x) for x in stack]
    assert kinds == ["T", 2.5, "T", "mul", "T", "mul", 1, "add", "assign"]
    assert stack[0] is C and stack[2] is A and stack[4] is B


def test_flat_vector_kernel(lib, fake_tensor):
    A, B, C = fake_tensor((1024, 128)), fake_tensor((1024, 128)), fake_tensor((1024, 128))
    src, info = _source(C, A * B + 1.5)
    assert info == {"flat": True, "vec": True, "threads": 256}
    assert "ld8" in src and "st8" in src
    _compiles(lib, src)


def test_flat_scalar_when_ragged(lib, fake_tensor):
    A, C = fake_tensor((3, 5)), fake_tensor((3, 5))
    src, info = _source(C, A + 1)
    assert info["flat"] and not info["vec"]
    _compiles(lib, src)


def test_batch_norm_shares_the_mean(lib, ops, fake_tensor):
    A = fake_tensor((4096, 128))
    expr = (A - ops.mean(A, axis=1)) / ops.sqrt(ops.var(A, axis=1) + 1e-3)
    src, info = _source(A, expr)
    assert not info["flat"] and info["threads"] == 32
    # two reductions only: sum(A) (shared by both means) and sum((A-mean)^2)
    assert src.count("const float rr") == 2
    assert "a0[ch][j]" in src and src.count("ld8(p0") == 1     # row read once, kept in registers
    _compiles(lib, src)


def test_reduction_axis_rules(ops, fake_tensor):
    A = fake_tensor((16, 16))
    with pytest.raises(ValueError):
        _source(A, ops.sum(A, axis=0) + ops.sum(A, axis=1))
    with pytest.raises(ValueError):
        _source(A, OpTreeNode.build("sum", A, None, axis=None))


def test_shape_mismatch_raises(fake_tensor):
    A, B = fake_tensor((4, 8)), fake_tensor((5, 8))
    C = fake_tensor((4, 8))
    with pytest.raises(TypeError):
        _source(C, A[:, 0:1] + B)   # broadcast forces the 2-D path, where 4 != 5 is an error


def test_non_2d_complex_op_raises(ops, fake_tensor):
    A = fake_tensor((4, 4, 4))
    O = fake_tensor((4, 1))
    with pytest.raises(ValueError):
        _source(O, ops.sum(A, axis=1))


@pytest.mark.parametrize("dtype", [np.float16, np.float32, np.int8, np.uint8, np.int16, np.uint16, np.int32, np.uint32])
def test_all_dtypes_compile(lib, fake_tensor, dtype):
    A, B, C = fake_tensor((64, 64), dtype), fake_tensor((64, 64), dtype), fake_tensor((64, 64), dtype)
    _compiles(lib, _source(C, A * B - A)[0])
    _compiles(lib, _source(C, A.T + B)[0])


def test_every_operator_compiles(lib, ops, fake_tensor):
    A, B, C = fake_tensor((64, 64)), fake_tensor((64, 64)), fake_tensor((64, 64))
    unary = [ops.negative, ops.sgn, ops.absolute, ops.sqrt, ops.square, ops.exp, ops.exp2, ops.log, ops.log2,
             ops.sig, ops.sig2, ops.tanh, ops.tanh2, ops.finite, ops.reciprocal]
    binary = [ops.add, ops.subtract, ops.multiply, ops.divide, ops.power, ops.equal, ops.not_equal, ops.less,
              ops.less_equal, ops.greater, ops.greater_equal, ops.maximum, ops.minimum]
    expr = A
    for f in unary:
        expr = f(expr)
    for f in binary:
        expr = f(expr, B)
    expr = ops.clip(expr, -1.0, 1.0)
    _compiles(lib, _source(C, expr)[0])


def test_reductions_compile(lib, ops, fake_tensor):
    A = fake_tensor((256, 5000))
    col = fake_tensor((256, 1), np.float32)
    row = fake_tensor((1, 5000), np.float32)
    idx = fake_tensor((256, 1), np.int32)
    for expr, out in ((ops.sum(A, axis=1), col), (ops.max(A, axis=1), col), (ops.min(A, axis=0), row),
                      (ops.argmax(A, axis=1), idx), (ops.argmin(A, axis=1), idx),
                      (ops.sum(A, axis=0), row)):
        src, info = _source(out, expr)
        _compiles(lib, src)
    assert _source(col, ops.sum(A, axis=1))[1]["threads"] == 1024   # long rows get a whole CTA


def test_rand_take_onehot_and_rounding_compile(lib, ops, fake_tensor):
    A, C = fake_tensor((128, 64)), fake_tensor((128, 64))
    _compiles(lib, _source(C, ops.rand() <= 0.5)[0])
    Csr = fake_tensor((128, 64), rounding=10)
    src, _ = _source(Csr, A * 3)
    assert "sr_bits" in src
    _compiles(lib, src)
    idx = fake_tensor((64,), np.int32)
    hot = fake_tensor((10, 64))
    _compiles(lib, _source(hot, OpTreeNode.build("onehot", None, None, idx=idx, axis=0))[0])
    rows = fake_tensor((32,), np.int32)
    taken = fake_tensor((32, 64))
    view = A[rows, :] if False else None   # fancy indexing with a device tensor builds a take view
    view = A.take(rows, 0)
    _compiles(lib, _source(taken, view * 2)[0])


def test_kernel_signature_is_shape_independent(fake_tensor):
    A, B = fake_tensor((64, 64)), fake_tensor((64, 64))
    A2, B2 = fake_tensor((128, 8)), fake_tensor((128, 8))
    p1 = float_ew._analyse(OpTreeNode({"op": "assign"}, A, B + 1).traverse([]))
    p2 = float_ew._analyse(OpTreeNode({"op": "assign"}, A2, B2 + 1).traverse([]))
    assert float_ew._signature(p1, True, 256, 0) == float_ew._signature(p2, True, 256, 0)
