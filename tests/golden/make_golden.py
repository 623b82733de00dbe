"""Generates tests/golden/*.npz by running the REFERENCE's own numpy validation code.

The reference's conv and pool checks live inline in benchmarks/conv_test.py and
benchmarks/pool_test.py, behind `import pycuda` and GPU launches. This script (run once, in a
container that has the reference checkout; the fixtures it writes are committed) executes those
two scripts unmodified except for:
  * the GPU modules (pycuda, nervanagpu) are replaced by stand-ins whose launches do nothing,
  * the hand-edited configuration lines at the top (layer shape, `cpu`, `ops`) are set to the
    case being generated, as a user of those scripts would do,
  * np.random.uniform is seeded and its draws are quantised to fp16-representable values, so the
    fp16 device kernels can consume exactly the same inputs.
The arrays the scripts compute on the CPU (cpuO / cpuB / cpuU) are stored with their inputs.

Usage: python tests/golden/make_golden.py <path of a checkout of the reference>
"""
import builtins
import functools
import os
import re
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle.reference_math import ConvDims, PoolDims  # noqa: E402  (shape bookkeeping only)


class _FakeDev(object):
    def __init__(self, shape):
        self.shape = tuple(shape)

    def get(self):
        return np.zeros(self.shape, dtype=np.float32)


class _FakeGPU(object):
    """Stands in for nervanagpu.NervanaGPU: layer objects carry dimensions, launches are no-ops."""

    def __init__(self, **kw):
        pass

    def conv_layer(self, dtype, *args):
        return ConvDims(*args)

    def pool_layer(self, dtype, op, *args):
        pd = PoolDims(*args)
        pd.op = op
        return pd

    def array(self, ary, dtype=None):
        return _FakeDev(ary.shape)

    def empty(self, shape, dtype=None):
        return _FakeDev(shape)

    zeros = empty

    def _noop(self, *a, **k):
        return None

    fprop_conv = bprop_conv = update_conv = fprop_pool = bprop_pool = _noop


class _Device(object):
    def name(self):
        return "reference numpy path (no device)"


class _Context(object):
    def get_device(self):
        return _Device()


class _Random(object):
    def __init__(self, seed):
        self.rs = np.random.RandomState(seed)

    def uniform(self, lo, hi, shape):
        return self.rs.uniform(lo, hi, shape).astype(np.float16).astype(np.float64)


class _NumpyProxy(object):
    """numpy with a seeded, fp16-quantising random.uniform."""

    def __init__(self, seed):
        self.random = _Random(seed)

    def __getattr__(self, name):
        return getattr(np, name)


def _run_reference_script(path, patches, seed):
    text = open(path).read()
    for pattern, repl in patches:
        text, n = re.subn(pattern, repl, text, count=1, flags=re.S)
        assert n == 1, "pattern not found in %s: %s" % (path, pattern)
    # GPU-only imports and numpy are provided through the namespace instead
    text = re.sub(r"^import numpy\s+as np$", "", text, flags=re.M)
    text = re.sub(r"^import pycuda\.driver as drv$", "", text, flags=re.M)
    text = re.sub(r"^from nervanagpu\s+import NervanaGPU$", "", text, flags=re.M)
    text = re.sub(r"^from pycuda\.autoinit import context$", "", text, flags=re.M)
    ns = {"np": _NumpyProxy(seed), "NervanaGPU": _FakeGPU, "context": _Context(), "drv": types.SimpleNamespace(),
          "__name__": "__reference__"}
    builtins.reduce = functools.reduce   # Python-2 builtin used by pool_test.py
    stdout, sys.stdout = sys.stdout, open(os.devnull, "w")   # the scripts print whole tensors
    try:
        exec(compile(text, path, "exec"), ns)
    except SystemExit:
        pass   # the scripts exit() after printing a mismatch against the (stand-in) device result
    finally:
        sys.stdout.close()
        sys.stdout = stdout
        del builtins.reduce
    return ns


CONV_CASES = {
    # name: (N, C, K, D, H, W, T, R, S, pad_d, pad_h, pad_w, str_d, str_h, str_w)
    "conv_3x3_pad1": (8, 5, 8, 1, 10, 9, 1, 3, 3, 0, 1, 1, 1, 1, 1),
    "conv_5x5_stride2_pad2": (8, 3, 16, 1, 13, 13, 1, 5, 5, 0, 2, 2, 1, 2, 2),
    "conv_3d": (8, 4, 8, 5, 6, 6, 3, 3, 3, 1, 1, 0, 1, 1, 1),
    "conv_16ch_n64": (64, 16, 64, 1, 5, 5, 1, 3, 3, 0, 1, 1, 1, 1, 1),
}

POOL_CASES = {
    # name: (N, C, D, H, W, J, T, R, S, pad_j, pad_d, pad_h, pad_w, str_j, str_d, str_h, str_w)
    "pool_3x3_stride2_overlap": (8, 4, 1, 9, 9, 1, 1, 3, 3, 0, 0, 0, 0, 1, 1, 2, 2),
    "pool_jtrs_2222": (8, 6, 4, 6, 6, 2, 2, 2, 2, 0, 0, 0, 0, 2, 2, 2, 2),
    "pool_featuremap_overlap": (32, 8, 1, 8, 8, 2, 1, 3, 3, 0, 0, 0, 0, 2, 1, 2, 2),
}


def _fmt(vals):
    return ",".join(str(v) for v in vals)


def make_conv(ref_root, name, cfg, seed):
    N, C, K, D, H, W, T, R, S, pd, ph, pw, sd, sh, sw = cfg
    patches = [
        (r'ops\s*=\s*set\(\("update",\)\)', 'ops  = set(("fprop","bprop","update"))'),
        (r"\ncpu\s*=\s*0", "\ncpu  = 1"),
        (r"conv = ng\.conv_layer\(.*?\)\s*# strides\n",
         "conv = ng.conv_layer(dtype, %s)\n" % _fmt(cfg)),
    ]
    ns = _run_reference_script(os.path.join(ref_root, "benchmarks", "conv_test.py"), patches, seed)
    cd = ns["conv"]
    out = {
        "cfg": np.array(cfg, dtype=np.int32),
        "I": ns["cpuI"][:-1, :].reshape(cd.dimI).astype(np.float16),
        "F": ns["cpuF"].reshape(cd.dimF).astype(np.float16),
        "E": ns["cpuE"].astype(np.float16),
        "O": ns["cpuO"].astype(np.float32),
        "gradI": ns["cpuB"][:-1, :].reshape(cd.dimI).astype(np.float32),
        "gradF": ns["cpuU"].reshape(cd.dimF).astype(np.float32),
    }
    # inputs were drawn fp16-representable, so the casts above are exact
    assert np.array_equal(out["I"].astype(np.float32), ns["cpuI"][:-1, :].reshape(cd.dimI))
    assert np.array_equal(out["E"].astype(np.float32), ns["cpuE"])
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print("wrote", name, {k: v.shape for k, v in out.items()})


def make_pool(ref_root, name, cfg, seed):
    patches = [
        (r"pool = ng\.pool_layer\(dtype,.*?\)\s*# strides\n",
         'pool = ng.pool_layer(dtype, "max", %s)\n' % _fmt(cfg)),
    ]
    ns = _run_reference_script(os.path.join(ref_root, "benchmarks", "pool_test.py"), patches, seed)
    pd = ns["pool"]
    out = {
        "cfg": np.array(cfg, dtype=np.int32),
        "I": ns["cpuI"].astype(np.float16),
        "O": ns["cpuO"].astype(np.float32),
        "gradI": ns["cpuB"].astype(np.float32),   # the script back-propagates its own output
    }
    assert out["I"].shape == pd.dimI
    assert np.array_equal(out["I"].astype(np.float32), ns["cpuI"])
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print("wrote", name, {k: v.shape for k, v in out.items()})


def main():
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    ref_root = sys.argv[1]
    for i, (name, cfg) in enumerate(sorted(CONV_CASES.items())):
        make_conv(ref_root, name, cfg, 100 + i)
    for i, (name, cfg) in enumerate(sorted(POOL_CASES.items())):
        make_pool(ref_root, name, cfg, 200 + i)


if __name__ == "__main__":
    main()
