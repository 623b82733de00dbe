"""ctypes binding of libnervana_b200.so (the C ABI declared in include/nervana_b200.h).

This is the only place that touches the shared library. There is no CPU fallback: if the
library is missing or the device is not an sm_100 GPU, calls raise.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libnervana_b200.so")

c_int, c_uint, c_float, c_size_t = ctypes.c_int, ctypes.c_uint, ctypes.c_float, ctypes.c_size_t
c_void_p, c_char_p, c_ulonglong, c_longlong = ctypes.c_void_p, ctypes.c_char_p, ctypes.c_ulonglong, ctypes.c_longlong
c_ubyte, c_ushort = ctypes.c_ubyte, ctypes.c_ushort

NG_PATH_AUTO, NG_PATH_TENSOR, NG_PATH_SIMT, NG_PATH_IM2COL = 0, 1, 2, 3

NG_ERRORS = {
    -1: "NG_ERR_INVALID_ARG", -2: "NG_ERR_UNSUPPORTED", -3: "NG_ERR_CUDA", -4: "NG_ERR_NVRTC",
    -5: "NG_ERR_NCCL", -6: "NG_ERR_TIMEOUT", -7: "NG_ERR_NOT_INITIALIZED", -8: "NG_ERR_TOO_LARGE",
}


class NervanaError(RuntimeError):
    def __init__(self, code, message):
        RuntimeError.__init__(self, "%s (%d): %s" % (NG_ERRORS.get(code, "NG_ERR"), code, message))
        self.code = code


class ConvDesc(ctypes.Structure):
    _fields_ = [(n, c_int) for n in
                "N C K D H W T R S pad_d pad_h pad_w str_d str_h str_w".split()]


class PoolDesc(ctypes.Structure):
    _fields_ = [(n, c_int) for n in
                "N C D H W J T R S pad_j pad_d pad_h pad_w str_j str_d str_h str_w".split()]


# name -> (restype, argtypes); every symbol include/nervana_b200.h declares
SIGNATURES = {
    "ng_last_error": (c_char_p, []),
    "ng_init": (c_int, [c_int]),
    "ng_device_count": (c_int, [ctypes.POINTER(c_int)]),
    "ng_sm_count": (c_int, [ctypes.POINTER(c_int)]),
    "ng_malloc": (c_int, [ctypes.POINTER(c_void_p), c_size_t]),
    "ng_free": (c_int, [c_void_p]),
    "ng_host_alloc": (c_int, [ctypes.POINTER(c_void_p), c_size_t]),
    "ng_host_free": (c_int, [c_void_p]),
    "ng_mem_info": (c_int, [ctypes.POINTER(c_size_t), ctypes.POINTER(c_size_t)]),
    "ng_memcpy_h2d_async": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p]),
    "ng_memcpy_d2h_async": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p]),
    "ng_memcpy_d2d_async": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p]),
    "ng_memset_d8_async": (c_int, [c_void_p, c_ubyte, c_size_t, c_void_p]),
    "ng_memset_d16_async": (c_int, [c_void_p, c_ushort, c_size_t, c_void_p]),
    "ng_memset_d32_async": (c_int, [c_void_p, c_uint, c_size_t, c_void_p]),
    "ng_stream_create": (c_int, [ctypes.POINTER(c_void_p)]),
    "ng_stream_destroy": (c_int, [c_void_p]),
    "ng_stream_sync": (c_int, [c_void_p]),
    "ng_stream_wait_event": (c_int, [c_void_p, c_void_p]),
    "ng_event_create": (c_int, [ctypes.POINTER(c_void_p)]),
    "ng_event_destroy": (c_int, [c_void_p]),
    "ng_event_record": (c_int, [c_void_p, c_void_p]),
    "ng_event_sync": (c_int, [c_void_p]),
    "ng_event_elapsed_ms": (c_int, [c_void_p, c_void_p, ctypes.POINTER(c_float)]),
    "ng_sync": (c_int, []),
    "ng_device_status": (c_int, [ctypes.POINTER(c_int)]),
    "ng_set_wait_limit_ns": (c_int, [c_ulonglong]),
    "ng_test_wait_expires": (c_int, [c_ulonglong, c_void_p, c_void_p]),
    "ng_static_scratch_status": (c_int, [ctypes.POINTER(c_int)]),
    "ng_launch_count": (c_int, [ctypes.POINTER(c_ulonglong)]),
    "ng_fallback_launch_count": (c_int, [ctypes.POINTER(c_ulonglong)]),
    "ng_tune": (c_int, [c_char_p, c_int]),
    "ng_graph_capture_begin": (c_int, [c_void_p]),
    "ng_graph_capture_end": (c_int, [c_void_p, ctypes.POINTER(c_void_p)]),
    "ng_graph_launch": (c_int, [c_void_p, c_void_p]),
    "ng_graph_destroy": (c_int, [c_void_p]),
    "ng_hgemm": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                         c_float, c_float, c_int, c_int, c_ulonglong, c_uint, c_void_p]),
    "ng_hgemm_simt": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                              c_float, c_float, c_int, c_int, c_ulonglong, c_uint, c_void_p]),
    "ng_hgemm_static_scratch": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                        c_int, c_int, c_float, c_float, c_int, c_int, c_ulonglong, c_uint,
                                        c_void_p]),
    "ng_hgemm_batched": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                 c_int, c_float, c_float, c_int, c_int, c_ulonglong, c_uint, c_int, c_int,
                                 c_longlong, c_longlong, c_longlong, c_void_p]),
    "ng_conv_output_dims": (c_int, [ctypes.POINTER(ConvDesc), ctypes.POINTER(c_int), ctypes.POINTER(c_int),
                                    ctypes.POINTER(c_int)]),
    "ng_conv_fprop": (c_int, [ctypes.POINTER(ConvDesc), c_void_p, c_void_p, c_void_p, c_float, c_int, c_int,
                              c_void_p]),
    "ng_conv_bprop": (c_int, [ctypes.POINTER(ConvDesc), c_void_p, c_void_p, c_void_p, c_float, c_int, c_void_p]),
    "ng_conv_update": (c_int, [ctypes.POINTER(ConvDesc), c_void_p, c_void_p, c_void_p, c_int, c_float, c_int,
                               c_void_p]),
    "ng_pool_output_dims": (c_int, [ctypes.POINTER(PoolDesc), ctypes.POINTER(c_int), ctypes.POINTER(c_int),
                                    ctypes.POINTER(c_int), ctypes.POINTER(c_int)]),
    "ng_pool_fprop": (c_int, [ctypes.POINTER(PoolDesc), c_int, c_void_p, c_void_p, c_void_p]),
    "ng_pool_bprop": (c_int, [ctypes.POINTER(PoolDesc), c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "ng_pool_bprop_relu": (c_int, [ctypes.POINTER(PoolDesc), c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "ng_pool_fprop_op": (c_int, [ctypes.POINTER(PoolDesc), c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "ng_pool_bprop_op": (c_int, [ctypes.POINTER(PoolDesc), c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "ng_pool_argmax_bytes": (c_int, [ctypes.POINTER(PoolDesc), c_int, ctypes.POINTER(c_size_t)]),
    "ng_pool_fprop_argmax": (c_int, [ctypes.POINTER(PoolDesc), c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "ng_pool_bprop_argmax": (c_int, [ctypes.POINTER(PoolDesc), c_int, c_void_p, c_void_p, c_void_p, c_int,
                                     c_void_p]),
    "ng_ew_compile": (c_int, [c_char_p, c_char_p, c_int, ctypes.POINTER(c_void_p)]),
    "ng_ew_compile_only": (c_int, [c_char_p, c_int]),
    "ng_ew_compile_log": (c_char_p, []),
    "ng_ew_launch": (c_int, [c_void_p, c_uint, c_uint, c_uint, c_uint, c_uint, c_uint, c_uint,
                             ctypes.POINTER(c_void_p), c_void_p]),
    "ng_ew_release": (c_int, [c_void_p]),
    "ng_comm_unique_id_bytes": (c_int, []),
    "ng_comm_unique_id": (c_int, [c_void_p]),
    "ng_comm_init": (c_int, [ctypes.POINTER(c_void_p), c_int, c_int, c_void_p]),
    "ng_comm_allreduce_f32": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p]),
    "ng_comm_async_error": (c_int, [c_void_p]),
    "ng_comm_destroy": (c_int, [c_void_p]),
    "ng_peer_handle_bytes": (c_int, []),
    "ng_peer_max_bytes": (c_size_t, []),
    "ng_peer_create": (c_int, [ctypes.POINTER(c_void_p), c_int, c_int, c_void_p]),
    "ng_peer_connect": (c_int, [c_void_p, c_void_p]),
    "ng_peer_sum_sgd_f32": (c_int, [c_void_p, c_void_p, c_void_p, c_size_t, c_float, c_void_p]),
    "ng_peer_destroy": (c_int, [c_void_p]),
    # the reference's own C interface (bool results)
    "nervana_loadKernels": (ctypes.c_bool, [c_char_p]),
    "nervana_unloadKernels": (ctypes.c_bool, []),
    "nervana_randStateSizeBytes": (c_size_t, []),
    "nervana_hgemm": (ctypes.c_bool, [c_void_p, c_void_p, c_void_p, ctypes.c_bool, ctypes.c_bool, c_int, c_int, c_int,
                                      c_int, c_int, c_int, c_float, c_float, c_void_p, ctypes.c_bool, ctypes.c_bool,
                                      c_void_p, c_int]),
    "nervana_hgemm_colmajor": (ctypes.c_bool, [c_void_p, c_void_p, c_void_p, ctypes.c_bool, ctypes.c_bool, c_int,
                                               c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p,
                                               ctypes.c_bool, ctypes.c_bool, c_void_p, c_int]),
    "nervana_sgemm": (ctypes.c_bool, [c_void_p, c_void_p, c_void_p, ctypes.c_bool, ctypes.c_bool, c_int, c_int, c_int,
                                      c_int, c_int, c_int, c_float, c_float, c_void_p, ctypes.c_bool, ctypes.c_bool,
                                      c_void_p, c_int]),
    "nervana_sgemm_colmajor": (ctypes.c_bool, [c_void_p, c_void_p, c_void_p, ctypes.c_bool, ctypes.c_bool, c_int,
                                               c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_void_p,
                                               ctypes.c_bool, ctypes.c_bool, c_void_p, c_int]),
}

_lib = None
_initialised = set()


def load():
    """dlopen the library and attach prototypes. No device is touched."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("%s not found: build it with `python -m nervanagpu_b200.build`" % LIB_PATH)
        lib = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


def check(rc):
    if rc != 0:
        raise NervanaError(rc, load().ng_last_error().decode("utf-8", "replace"))


def init(device=None):
    """Select and initialise a device (default: LOCAL_RANK or 0). Idempotent per device."""
    lib = load()
    if device is None:
        device = int(os.environ.get("NERVANA_DEVICE", os.environ.get("LOCAL_RANK", "0")))
    if device not in _initialised:
        check(lib.ng_init(device))
        _initialised.add(device)
    return lib


def sm_count():
    n = c_int()
    check(init().ng_sm_count(ctypes.byref(n)))
    return n.value
