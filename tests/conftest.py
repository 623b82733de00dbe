import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) device")


def _have_gpu():
    try:
        from nervanagpu_b200 import _lib
        import ctypes
        n = ctypes.c_int(0)
        return _lib.load().ng_device_count(ctypes.byref(n)) == 0 and n.value > 0
    except Exception:
        return False


@pytest.fixture(scope="session")
def ng():
    """One NervanaGPU backend for the whole session (device 0)."""
    from nervanagpu_b200 import NervanaGPU
    return NervanaGPU(stochastic_round=False, bench=False)


@pytest.fixture(scope="session")
def lib():
    from nervanagpu_b200 import _lib
    return _lib.load()


class FakeBackend(object):
    """Stands in for NervanaGPU in host-only tests: tensors are given fake device addresses."""
    stream = None
    bench = False
    round_mode = 0


@pytest.fixture()
def fake_tensor():
    import numpy as np
    from nervanagpu_b200.nervanagpu import GPUTensor
    counter = [1 << 20]

    def make(shape, dtype=np.float16, rounding=0):
        counter[0] += 1 << 24
        return GPUTensor(FakeBackend(), shape, dtype=dtype, gpudata=counter[0], rounding=rounding)
    return make
