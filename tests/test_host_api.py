"""Host-only tests: the C-ABI library loads and exports every declared symbol; GPUTensor view
bookkeeping; layer dimension formulas. No device is touched."""
import os
import re

import numpy as np
import pytest

from nervanagpu_b200 import _lib
from nervanagpu_b200.layers import ConvLayer, PoolLayer, FullLayer, DataLayer, Layer
from nervanagpu_b200.nervanagpu import GPUTensor, _contiguous_strides

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "nervana_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b((?:ng|nervana)_[A-Za-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(lib):
    names = _declared_symbols()
    assert len(names) > 40
    for name in names:
        assert hasattr(lib, name), name
        assert name in _lib.SIGNATURES, "no ctypes prototype for %s" % name
    for name in _lib.SIGNATURES:
        assert name in names, "%s is bound but not declared in the header" % name


def test_descriptor_structs_match_header():
    assert [f[0] for f in _lib.ConvDesc._fields_] == "N C K D H W T R S pad_d pad_h pad_w str_d str_h str_w".split()
    assert len(_lib.PoolDesc._fields_) == 17


def test_strides_views_and_transpose(fake_tensor):
    A = fake_tensor((6, 8, 10))
    assert A.strides == (80, 10, 1) and A.is_contiguous and A.nbytes == 960
    v = A[2:5, :, 3]
    assert v.shape == (3, 8) and v.strides == (80, 10) and v.ptr == A.ptr + (2 * 80 + 3) * 2
    assert not v.is_contiguous and v.base is A
    assert A[1].shape == (8, 10) and A[1].ptr == A.ptr + 160
    assert A[..., 4].shape == (6, 8)
    assert A[::2].shape == (3, 8, 10) and A[::2].strides == (160, 10, 1)
    assert A[-1, -1, -1].ptr == A.ptr + (A.size - 1) * 2
    M = fake_tensor((4, 7))
    T = M.T
    assert T.shape == (7, 4) and T.strides == (1, 7) and T.is_trans and not T.T.is_trans
    B = A.T                       # batched: outer dim kept, inner two reversed
    assert B.shape == (6, 10, 8) and B.strides == (80, 1, 10)
    assert A[:] is A


def test_index_errors(fake_tensor):
    A = fake_tensor((4, 5))
    with pytest.raises(IndexError):
        A[4]
    with pytest.raises(IndexError):
        A[..., ..., 0]
    with pytest.raises(IndexError):
        A["x"]
    with pytest.raises(IndexError):
        A[fake_tensor((2, 2), np.int32), :]       # index tensors must be one-dimensional
    with pytest.raises(IndexError):
        A[fake_tensor((2,), np.uint8), :]         # and int32
    with pytest.raises(IndexError):
        A[fake_tensor((2,), np.int32), fake_tensor((2,), np.int32)]


def test_reshape_and_share(fake_tensor):
    A = fake_tensor((4, 6))
    R = A.reshape(3, 8)
    assert R.shape == (3, 8) and R.ptr == A.ptr and R.base is A
    assert A.reshape((4, 6)) is A
    with pytest.raises(ValueError):
        A.reshape(5, 5)
    with pytest.raises(TypeError):
        A[:, 1:3].reshape(8)
    S = A.share((2, 3), dtype=np.float32)
    assert S.dtype == np.float32 and S.shape == (2, 3)
    with pytest.raises(ValueError):
        A.share((5, 5))
    assert _contiguous_strides(()) == () and _contiguous_strides((3,)) == (1,)


def test_dtype_whitelist(fake_tensor):
    for dt in (np.float16, np.float32, np.uint8, np.int8, np.uint16, np.int16, np.uint32, np.int32):
        assert fake_tensor((2, 2), dt).dtype == np.dtype(dt)
    with pytest.raises(AssertionError):
        fake_tensor((2, 2), np.float64)


def test_conv_layer_dimensions():
    # BASELINE config 3 (AlexNet) and config 5 (3-D) shapes
    l1 = ConvLayer(None, np.float16, 128, 3, 64, 1, 224, 224, 1, 11, 11, 0, 2, 2, 1, 4, 4)
    assert l1.MPQ == (1, 55, 55) and l1.dimO == (64, 1, 55, 55, 128) and l1.dimF == (3, 1, 11, 11, 64)
    assert l1.flops == 55 * 55 * 64 * 128 * 3 * 121 * 2.0 and l1.nOut == 55 * 55 * 64
    assert l1.dtypeU is np.float32
    l2 = ConvLayer(None, np.float16, 128, 64, 192, 1, 27, 27, 1, 5, 5, 0, 2, 2)
    assert l2.MPQ == (1, 27, 27) and l2.sizeF == 64 * 25 * 192
    l5 = ConvLayer(None, np.float16, 32, 64, 64, 16, 56, 56, 3, 3, 3, 1, 1, 1)
    assert l5.MPQ == (16, 56, 56) and abs(l5.flops - 355.14e9) < 0.01e9
    with pytest.raises(AssertionError):
        ConvLayer(None, np.float16, 12, 3, 64, 1, 8, 8, 1, 3, 3)
    assert (l1.desc.N, l1.desc.str_w, l1.desc.pad_h) == (128, 4, 2)


def test_pool_layer_dimensions():
    p = PoolLayer(None, np.float16, "max", 128, 64, 1, 55, 55, 1, 1, 3, 3, str_h=2, str_w=2)
    assert p.dimO == (64, 1, 27, 27, 128) and p.overlap == 4.0
    p2 = PoolLayer(None, np.float16, "max", 32, 64, 16, 56, 56, 2, 2, 2, 2)
    assert p2.dimO == (32, 8, 28, 28, 32) and p2.overlap == 0.0 and p2.strides == (2, 2, 2, 2)


def test_layer_create_propagates_dimensions():
    confs = [
        {"layer": DataLayer, "N": 64, "C": 3, "H": 32, "W": 32},
        {"layer": ConvLayer, "common": {"R": 3, "S": 3, "pad_h": 1, "pad_w": 1}, "K": 16},
        {"layer": PoolLayer, "op": "max", "R": 2, "S": 2},
        {"layer": FullLayer, "nOut": 100},
    ]
    prev = None
    layers = []
    for conf in confs:
        prev = Layer.create(None, conf, prev, np.float16)
        layers.append(prev)
    assert layers[1].dimI == (3, 1, 32, 32, 64) and layers[1].dimO == (16, 1, 32, 32, 64)
    assert layers[2].dimO == (16, 1, 16, 16, 64)
    assert layers[3].nIn == 16 * 16 * 16 and layers[3].dimF == (100, 4096)


def test_network_tables_build_with_consistent_shapes():
    """Every network of the whole-network driver, created through Layer.create without a device:
    map sizes follow the published architectures and every Inception module concatenates its
    four branches."""
    from nervanagpu_b200 import convnet_benchmarks as cb
    from nervanagpu_b200.layers import Inception
    for name, (_, confs) in cb.NETWORKS.items():
        prev, layers = None, []
        for conf in confs:
            prev = Layer.create(None, conf, prev, np.float16)
            layers.append(prev)
        assert layers[-1].nOut == 1000, name
        for a, b in zip(layers, layers[1:]):
            assert b.sizeI == a.sizeO, (name, str(a), str(b))
    _, confs = cb.NETWORKS["GoogLeNet1"]
    prev, modules = None, []
    for conf in confs:
        prev = Layer.create(None, conf, prev, np.float16)
        if isinstance(prev, Inception):
            modules.append(prev)
    assert [m.K for m in modules] == [256, 480, 512, 512, 512, 528, 832, 832, 1024]
    assert [m.P for m in modules] == [28, 28, 14, 14, 14, 14, 14, 7, 7]
    first = modules[0]
    assert [len(part) for part in first.partitions] == [1, 2, 2, 2]
    assert first.flops == sum(l.flops for part in first.partitions for l in part) > 0
