"""B200 (sm_100a) implementation of the nervanagpu compute core behind its Python API."""
from .nervanagpu import NervanaGPU, GPUTensor, OpTreeNode  # noqa: F401
from .layers import (Layer, DataLayer, FullLayer, ConvLayer, DeconvLayer, PoolLayer)  # noqa: F401

__version__ = "0.1.0"
