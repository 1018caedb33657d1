"""ctypes binding of libsmall_b200.so (the C ABI declared in include/small_b200.h).

There is no fallback: if the library is missing or a call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "lib", "libsmall_b200.so")

OK, INVALID_ARGUMENT, CUDA_ERROR, OUT_OF_MEMORY, DEVICE_TIMEOUT = range(5)
ACT_NONE, ACT_RELU, ACT_LEAKY = 0, 1, 2


class Layer(C.Structure):
    """small_b200_layer"""
    _fields_ = ([(n, C.c_int32) for n in
                 ("N", "C", "K", "H", "W", "Fh", "Fw", "stride",
                  "pad_t", "pad_b", "pad_l", "pad_r", "accumulate", "act")]
                + [("slope", C.c_float)]
                + [(n, C.c_int32) for n in
                   ("zero_in", "zero_filt", "lshift", "rshift", "multiplier", "k_zero", "stride_h")])

    def out_hw(self):
        ho = max((self.H + self.pad_t + self.pad_b - self.Fh) // (self.stride_h or self.stride) + 1, 0)
        wo = max((self.W + self.pad_l + self.pad_r - self.Fw) // self.stride + 1, 0)
        return ho, wo


class SmallB200Error(RuntimeError):
    pass


_lib = None

_VP, _I32, _I64, _SZ, _F = C.c_void_p, C.c_int32, C.c_int64, C.c_size_t, C.c_float
_LP = C.POINTER(Layer)

# name -> argtypes; every function returns int except the two noted below
SIGNATURES = {
    "small_b200_device_count": [C.POINTER(C.c_int)],
    "small_b200_set_device": [C.c_int],
    "small_b200_device_status": [C.POINTER(C.c_int)],
    "small_b200_selftest_bounded_wait": [C.c_uint32, _VP],
    "small_b200_peak_probe": [C.c_int, C.POINTER(C.c_double)],
    "small_b200_malloc": [_SZ, C.POINTER(_VP)],
    "small_b200_malloc_managed": [_SZ, C.POINTER(_VP)],
    "small_b200_malloc_host": [_SZ, C.POINTER(_VP)],
    "small_b200_malloc_host_upload": [_SZ, C.POINTER(_VP)],
    "small_b200_free": [_VP],
    "small_b200_free_host": [_VP],
    "small_b200_memcpy_h2d": [_VP, _VP, _SZ, _VP],
    "small_b200_memcpy_d2h": [_VP, _VP, _SZ, _VP],
    "small_b200_memcpy_d2d": [_VP, _VP, _SZ, _VP],
    "small_b200_prefetch": [_VP, _SZ, _VP],
    "small_b200_stream_create": [C.POINTER(_VP)],
    "small_b200_stream_destroy": [_VP],
    "small_b200_stream_sync": [_VP],
    "small_b200_device_sync": [],
    "small_b200_graph_begin": [_VP],
    "small_b200_graph_end": [_VP, C.POINTER(_VP)],
    "small_b200_graph_launch": [_VP, _VP],
    "small_b200_graph_destroy": [_VP],
    "small_b200_conv2d_f32": [_LP, _VP, _VP, _VP, _VP, _VP],
    "small_b200_conv2d_maxpool_f32_supported": [_LP, _LP],
    "small_b200_conv2d_maxpool_f32": [_LP, _LP, _VP, _VP, _VP, _VP, _VP],
    "small_b200_conv2d_maxpool_f32_tf32x3_supported": [_LP, _LP],
    "small_b200_conv2d_maxpool_f32_tf32x3": [_LP, _LP, _VP, _VP, _VP, _VP, _VP],
    "small_b200_conv2d_f32_tf32x3_supported": [_LP],
    "small_b200_conv2d_f32_tf32x3_preferred": [_LP],
    "small_b200_filter_prepare_tf32x3": [_LP, _VP, _VP, _VP],
    "small_b200_conv2d_f32_tf32x3": [_LP, _VP, _VP, _VP, _VP, _VP],
    "small_b200_conv2d_f32_tf32x3_noalloc": [_LP, _VP, _VP, _VP, _VP, _VP],
    "small_b200_dwconv2d_f32": [_LP, _VP, _VP, _VP, _VP, _VP],
    "small_b200_groupconv2d_f32": [_LP, C.c_int32, _VP, _VP, _VP, _VP, _VP],
    "small_b200_blockconv2d_f32": [_LP, C.c_int32, _VP, _VP, _VP, _VP, _VP],
    "small_b200_maxpool2d_f32": [_LP, _VP, _VP, _VP],
    "small_b200_avgpool2d_f32": [_LP, _VP, _VP, _VP],
    "small_b200_relu_f32": [_I64, _VP, _VP, _VP],
    "small_b200_leaky_relu_f32": [_I64, _VP, _F, _VP, _VP],
    "small_b200_accum_f32": [_I64, _VP, _VP, _VP],
    "small_b200_scale_f32": [_I64, _VP, _F, _VP, _VP],
    "small_b200_bias_f32": [_I32, _I32, _I32, _I32, _VP, _I32, _VP, _VP],
    "small_b200_upsample2d_f32": [_I32, _I32, _I32, _I32, _VP, _VP, _VP],
    "small_b200_upsample1d_f32": [_I32, _I32, _I32, _I32, _VP, _VP, _VP],
    "small_b200_softmax_f32": [_I32, _I64, _VP, _VP, _VP],
    "small_b200_concat": [_I32, _SZ, _VP, _SZ, _VP, _VP, _VP],
    "small_b200_conv_weights_prepare_f32": [_I32, _I32, _I32, _I32, _I32, _VP, _VP, _VP, _VP, _VP, _VP, _F, _VP, _VP, _VP],
    "small_b200_yolo_decode_f32": [_I32, _I32, _I32, _I32, _I32, _I32, _F, _VP, _VP, _VP, _VP],
    "small_b200_nms_f32": [_VP, _I32, _I32, _F, _F, _I32, _VP, _I32, _VP, _VP, _VP],
    "small_b200_conv2d_u8": [_LP, _VP, _VP, _VP, _VP, _VP],
    "small_b200_conv2d_u8_cuda_cores": [_LP, _VP, _VP, _VP, _VP, _VP],
    "small_b200_conv2d_u8_tensor_core": [_LP, _VP, _VP, _VP, _VP, _VP],
    "small_b200_dwconv2d_u8": [_LP, _VP, _VP, _VP, _VP, _VP],
    "small_b200_conv2d_dwconv2d_u8_supported": [_LP, _LP],
    "small_b200_conv2d_dwconv2d_u8": [_LP, _LP, _VP, _VP, _VP, _VP, _VP, _VP, _VP],
    "small_b200_conv2d_avgpool_dense_u8_supported": [_LP, _LP, _LP],
    "small_b200_conv2d_avgpool_dense_u8": [_LP, _LP, _LP, _VP, _VP, _VP, _VP, _VP, _VP, _VP],
    "small_b200_groupconv2d_u8": [_LP, C.c_int32, _VP, _VP, _VP, _VP, _VP],
    "small_b200_maxpool2d_u8": [_LP, _VP, _VP, _VP],
    "small_b200_avgpool2d_u8": [_LP, _VP, _VP, _VP],
    "small_b200_relu_u8": [_I64, _LP, _VP, _VP, _VP],
}
OTHER = {"small_b200_last_error": ([], C.c_char_p), "small_b200_launch_count": ([], C.c_uint64),
         "small_b200_nms_scratch_bytes": ([C.c_int32], C.c_size_t)}


def exported_names():
    return sorted(list(SIGNATURES) + list(OTHER))


def lib():
    """Load the library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise SmallB200Error(
                f"{LIB_PATH} not found: build it with `python -m smallframework_b200.build` "
                "(there is no CPU fallback)")
        l = C.CDLL(LIB_PATH)
        for name, args in SIGNATURES.items():
            fn = getattr(l, name)
            fn.argtypes = args
            fn.restype = C.c_int
        for name, (args, res) in OTHER.items():
            fn = getattr(l, name)
            fn.argtypes = args
            fn.restype = res
        _lib = l
    return _lib


def check(rc: int):
    """Translate a return code the way the C++ platform headers do."""
    if rc == OK:
        return
    msg = lib().small_b200_last_error().decode()
    if rc == INVALID_ARGUMENT:
        raise ValueError(msg)  # std::invalid_argument in the reference
    if rc == OUT_OF_MEMORY:
        raise MemoryError(msg)  # std::bad_alloc
    raise SmallB200Error(f"[{rc}] {msg}")


def device_status() -> int:
    """Synchronise and raise if a kernel gave up on a bounded wait."""
    v = C.c_int(0)
    check(lib().small_b200_device_status(C.byref(v)))
    return v.value


def launch_count() -> int:
    return int(lib().small_b200_launch_count())
