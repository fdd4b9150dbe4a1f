"""ctypes binding of ``liboccamy_dnn.so`` -- the operator runtime behind the C ABI of
``include/occamy_dnn_api.h``.

There is no Python or CPU implementation behind this module: if the native library has
not been built, or no sm_100 GPU is present, it raises.  Device memory is obtained from
the ABI's own allocator (``wrapDNNMalloc``), so callers need neither torch nor numpy
device arrays.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "liboccamy_dnn.so")

_i64p = C.POINTER(C.c_int64)
_f32p = C.c_void_p  # device pointers travel as opaque addresses
_lib = None

# name -> (restype, argtypes); the order and meaning are those of include/occamy_dnn_api.h
_SIGNATURES = {
    "wrapDNNMalloc": (C.c_int, [C.POINTER(C.c_void_p), C.c_size_t]),
    "wrapDNNMemPoolInit": (C.c_int, [C.POINTER(C.c_void_p), C.c_size_t]),
    "wrapDNNMemOffset": (C.c_int, [C.POINTER(C.c_void_p), C.c_void_p, C.c_size_t, C.c_size_t]),
    "wrapDNNMemcpy": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]),
    "wrapDNNDealloc": (C.c_int, [C.c_void_p]),
    "cudnnCreate": (C.c_int, [C.POINTER(C.c_void_p)]),
    "cudnnDestroy": (C.c_int, [C.c_void_p]),
    "DNNConvFunc": (C.c_void_p, [C.c_void_p, _f32p, _i64p, _f32p, _i64p, _f32p, C.c_int64,
                                 C.c_int64, C.c_int64, _i64p, _i64p, _f32p]),
    "DNNConvBiasActivFunc": (C.c_void_p, [C.c_void_p, _f32p, _i64p, _f32p, _i64p, _f32p, _i64p,
                                          _f32p, C.c_int64, C.c_int64, _i64p, _i64p, C.c_int64,
                                          _f32p]),
    "DNNActiveFunc": (C.c_void_p, [C.c_void_p, _f32p, _i64p, C.c_int32, _f32p]),
    "DNNTensorOpFunc": (C.c_void_p, [C.c_void_p, C.c_int64, _f32p, _i64p, C.c_int32, _f32p, _i64p,
                                     C.c_int32, _f32p, _i64p, C.c_int32, C.c_float]),
    "CUDAClipFunc": (C.c_void_p, [_f32p, _f32p, _i64p, C.c_float, C.c_float, C.c_int64]),
    "DNNMaxPoolFunc": (C.c_void_p, [C.c_void_p, _f32p, _i64p, _f32p, _i64p, _i64p, _i64p, _i64p]),
    "DNNAveragePoolFunc": (C.c_void_p, [C.c_void_p, _f32p, _i64p, _f32p, _i64p, _i64p, _i64p,
                                        _i64p]),
    "DNNReduceFunc": (C.c_void_p, [C.c_void_p, C.c_int32, _f32p, _i64p, _f32p, _i64p, C.c_int32]),
    "CUBLASMatmul2dFunc": (C.c_void_p, [C.c_int64, _f32p, _i64p, _f32p, _i64p, _f32p, _i64p, _f32p,
                                        _i64p, C.c_float, C.c_float, C.c_int64, C.c_int64]),
    "CUDASoftmaxFunc": (C.c_void_p, [_f32p, _i64p, _f32p, _i64p, C.c_int64, C.c_int64]),
    "CUDAFlattenFunc": (C.c_void_p, [_f32p, _i64p, _f32p, _i64p, C.c_int32, C.c_int64]),
    "CUDAReshapeFunc": (C.c_void_p, [_f32p, _i64p, C.c_int64, _f32p]),
    "CUDACastI64toFloatFunc": (C.c_void_p, [C.c_void_p, _f32p, _i64p, C.c_int64]),
    "CUDAConcatFloatFunc": (C.c_void_p, [C.POINTER(C.c_void_p), C.POINTER(_i64p), _f32p, _i64p,
                                         C.c_int64, C.c_int64, C.c_int32]),
    "CUDAConcatInt64Func": (C.c_void_p, [C.POINTER(C.c_void_p), C.POINTER(_i64p), C.c_void_p,
                                         _i64p, C.c_int64, C.c_int64, C.c_int32]),
    "CUDAErfFunc": (C.c_void_p, [_f32p, _f32p, _i64p, C.c_int64]),
    "CUDAExpandInt64Func": (C.c_void_p, [C.c_void_p, _i64p, C.c_int64, C.c_void_p, _i64p,
                                         C.c_void_p, _i64p]),
    "CUDAGatherFloatFunc": (C.c_void_p, [_f32p, _i64p, C.c_int64, _f32p, _i64p, C.c_int64,
                                         C.c_void_p, _i64p, C.c_int64, C.c_int64]),
    "CUDAGatherInt64Func": (C.c_void_p, [C.c_void_p, _i64p, C.c_int64, C.c_void_p, _i64p,
                                         C.c_int64, C.c_void_p, _i64p, C.c_int64, C.c_int64]),
    "CUDALeakyReluFunc": (C.c_void_p, [_f32p, _f32p, _i64p, C.c_float, C.c_int64]),
    "CUDAMatmulNdFunc": (C.c_void_p, [_f32p, _i64p, C.c_int32, _f32p, _i64p, C.c_int32, _f32p,
                                      _i64p, C.c_int32]),
    "CUDANegativeFunc": (C.c_void_p, [_f32p, _f32p, _i64p, C.c_int64]),
    "CUDAReciprocalFunc": (C.c_void_p, [_f32p, _f32p, _i64p, C.c_int64]),
    "CUDANonZeroFloatFunc": (C.c_void_p, [_f32p, _i64p, _f32p, _i64p, C.c_int64]),
    "CUDANonZeroInt64Func": (C.c_void_p, [C.c_void_p, _i64p, C.c_void_p, _i64p, C.c_int64]),
    "CUDAPReluFunc": (C.c_void_p, [_f32p, _f32p, _i64p, _f32p, C.c_int64]),
    "CUDAPowFunc": (C.c_void_p, [_f32p, _f32p, _f32p, _i64p, C.c_int64]),
    "CUDASqueezeFloatFunc": (C.c_void_p, [_f32p, _i64p, _f32p, _i64p, C.c_int32, C.c_int64]),
    "CUDASqueezeInt64Func": (C.c_void_p, [C.c_void_p, _i64p, C.c_void_p, _i64p, C.c_int32,
                                          C.c_int64]),
    "CUDAUnsqueezeFloatFunc": (C.c_void_p, [_f32p, _i64p, _f32p, _i64p, C.c_int32, C.c_int64]),
    "CUDAUnsqueezeInt64Func": (C.c_void_p, [C.c_void_p, _i64p, C.c_void_p, _i64p, C.c_int32,
                                            C.c_int64]),
    "occamy_set_math_mode": (None, [C.c_int]),
    "occamy_get_math_mode": (C.c_int, []),
    "occamy_last_error": (C.c_int, [C.c_int]),
    "occamy_synchronize": (C.c_int, []),
    "occamy_stream": (C.c_void_p, []),
    "occamy_selftest_bounded_wait": (None, []),
    "occamy_get_counters": (None, [_i64p]),
    "occamy_clear_weight_cache": (None, []),
    "occamy_set_weight_cache": (None, [C.c_int]),
    "occamy_set_fp32_tensor_cores": (None, [C.c_int]),
    "occamy_conv_bias_act_noalloc": (C.c_int, [_f32p, _i64p, _f32p, _i64p, _f32p, _i64p, _i64p,
                                               C.c_int64, _f32p, C.c_void_p]),
    "occamy_noalloc_last_error": (C.c_int, [C.c_int]),
    "occamy_noalloc_capacity": (C.c_int64, []),
    "occamy_fused_chains": (C.c_int64, []),
    "occamy_set_cross_call_fusion": (None, [C.c_int]),
    "occamy_profile_begin": (None, []),
    "occamy_profile_end": (C.c_int, [C.POINTER(C.c_float), C.c_int]),
}
for _r in (2, 3, 4, 6):
    _SIGNATURES[f"CUDATranspose{_r}DFloatFunc"] = (C.c_void_p, [_f32p, _i64p, _f32p, _i64p, _i64p,
                                                                C.c_int64])
    _SIGNATURES[f"CUDATranspose{_r}DInt64Func"] = (C.c_void_p, [C.c_void_p, _i64p, C.c_void_p,
                                                                _i64p, _i64p, C.c_int64])

MATH_FP32, MATH_BF16, MATH_F16 = 0, 1, 2
COUNTER_NAMES = ("launches", "h2d_bytes", "h2d_skipped_bytes", "pool_hwm_bytes", "tc_launches",
                 "materializations", "tmap_encodes", "simt_launches")


def abi_symbols():
    """Every symbol name the public header declares and this module binds."""
    return sorted(_SIGNATURES)


def load_library(path: str = LIB_PATH):
    """dlopen the runtime and attach signatures; does not touch the GPU."""
    if not os.path.exists(path):
        raise RuntimeError(
            f"{path} is missing: build it with `python -m occamy_b200.build` "
            "(there is no Python/CPU fallback for the operator runtime)")
    lib = C.CDLL(path, mode=os.RTLD_LOCAL | os.RTLD_NOW)
    for name, (res, args) in _SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = ABI symbol missing from the build
        fn.restype = res
        fn.argtypes = args
    return lib


def lib():
    global _lib
    if _lib is None:
        _lib = load_library()
    return _lib


def dims(d):
    return (C.c_int64 * len(d))(*[int(v) for v in d])


def set_math_mode(mode: int):
    lib().occamy_set_math_mode(int(mode))


def synchronize():
    e = lib().occamy_synchronize()
    if e:
        raise RuntimeError(f"occamy_synchronize: CUDA error {e}")


def last_error(clear: bool = True) -> int:
    return lib().occamy_last_error(1 if clear else 0)


def counters() -> dict:
    out = (C.c_int64 * 8)()
    lib().occamy_get_counters(out)
    return dict(zip(COUNTER_NAMES, [int(v) for v in out]))


class DeviceBuffer:
    """A device allocation from the ABI's allocator (zero-filled, as the ABI promises)."""

    def __init__(self, nbytes: int):
        self.nbytes = int(nbytes)
        p = C.c_void_p()
        lib().wrapDNNMalloc(C.byref(p), self.nbytes)
        self.ptr = p.value

    @classmethod
    def from_numpy(cls, a: np.ndarray) -> "DeviceBuffer":
        a = np.ascontiguousarray(a)
        buf = cls(a.nbytes)
        if a.nbytes:
            # The library keeps the host address as the identity of an uploaded constant, so
            # the array must outlive the buffer.
            buf._keep = a
            lib().wrapDNNMemcpy(buf.ptr, a.ctypes.data, a.nbytes, 1, None)
        return buf

    def to_numpy(self, shape, dtype=np.float32) -> np.ndarray:
        out = np.empty(shape, dtype)
        if out.nbytes:
            lib().wrapDNNMemcpy(out.ctypes.data, self.ptr, out.nbytes, 2, None)
        return out

    def free(self):
        if self.ptr:
            lib().wrapDNNDealloc(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass
