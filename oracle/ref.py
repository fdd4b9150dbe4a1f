"""numpy front-end of the CPU oracle (``occamy_oracle.c``) -- TEST INFRASTRUCTURE.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import this module; the product (``occamy_b200``) never does.  Each function
mirrors one runtime symbol of the reference ABI on host fp32 NCHW arrays and
returns a new array.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build as _build

_lib = None
_i64p = C.POINTER(C.c_int64)
_f32p = C.POINTER(C.c_float)


def lib():
    global _lib
    if _lib is None:
        path = _build.ORACLE_SO
        if not os.path.exists(path):
            path = _build.build_oracle()
        _lib = C.CDLL(path)
    return _lib


def _fp(a):
    return a.ctypes.data_as(_f32p)


def _dims(d):
    return (C.c_int64 * len(d))(*[int(v) for v in d])


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def conv_out_hw(H, W, R, S, pad, stride):
    return (H + 2 * pad[0] - R) // stride[0] + 1, (W + 2 * pad[1] - S) // stride[1] + 1


def conv2d(x, w, bias=None, pads=(0, 0), strides=(1, 1), groups=1, act=5, lo=0.0, hi=0.0,
           f64=False):
    """DNNConvFunc / DNNConvBiasActivFunc. act: 1 ReLU, 3 clip[lo,hi], 5 identity."""
    x, w = _f32(x), _f32(w)
    N, Cc, H, W = x.shape
    K, Cg, R, S = w.shape
    assert Cg * groups == Cc, (x.shape, w.shape, groups)
    P, Q = conv_out_hw(H, W, R, S, pads, strides)
    y = np.empty((N, K, P, Q), np.float32)
    b = _f32(bias).reshape(-1) if bias is not None else None
    fn = lib().occ_conv2d_f64 if f64 else lib().occ_conv2d
    fn(_fp(x), _fp(w), _fp(b) if b is not None else None, _fp(y),
       *[C.c_int64(int(v)) for v in (N, Cc, H, W, K, R, S, groups, pads[0], pads[1],
                                     strides[0], strides[1])],
       C.c_int(int(act)), C.c_float(lo), C.c_float(hi))
    return y


def tensor_op(mode, A, B, biasB=1.0):
    """DNNTensorOpFunc: 0 add, 1 mul, 4 sqrt; B broadcast where its extent is 1."""
    A, B = _f32(A), _f32(B)
    dimB = [1] * (A.ndim - B.ndim) + list(B.shape)
    out = np.empty_like(A)
    lib().occ_tensor_op(C.c_int64(mode), _fp(A), _dims(A.shape), _fp(B), _dims(dimB), _fp(out),
                        C.c_int(A.ndim), C.c_float(biasB))
    return out


def activation(x, mode=1):
    x = _f32(x)
    y = np.empty_like(x)
    lib().occ_activation(_fp(x), _fp(y), C.c_int64(x.size), C.c_int(mode))
    return y


def clip(x, lo, hi):
    x = _f32(x)
    y = np.empty_like(x)
    lib().occ_clip(_fp(x), _fp(y), C.c_int64(x.size), C.c_float(lo), C.c_float(hi))
    return y


def pool_out_hw(H, W, kernel, pads, strides):
    return ((H + 2 * pads[0] - kernel[0]) // strides[0] + 1,
            (W + 2 * pads[1] - kernel[1]) // strides[1] + 1)


def pool2d(x, kernel, pads=(0, 0), strides=(1, 1), avg=False, count_include_pad=True):
    """DNNMaxPoolFunc / DNNAveragePoolFunc; pads = (h_begin, w_begin)."""
    x = _f32(x)
    N, Cc, H, W = x.shape
    P, Q = pool_out_hw(H, W, kernel, pads, strides)
    y = np.empty((N, Cc, P, Q), np.float32)
    lib().occ_pool2d(_fp(x), _fp(y),
                     *[C.c_int64(int(v)) for v in (N, Cc, H, W, P, Q, kernel[0], kernel[1],
                                                   pads[0], pads[1], strides[0], strides[1])],
                     C.c_int(int(avg)), C.c_int(int(count_include_pad)))
    return y


def reduce_mean(x, out_shape):
    """DNNReduceFunc mode 5: mean over the axes whose output extent is 1."""
    x = _f32(x)
    y = np.empty(tuple(out_shape), np.float32)
    lib().occ_reduce_mean(_fp(x), _dims(x.shape), _fp(y), _dims(out_shape), C.c_int(x.ndim))
    return y


def matmul2d(A, B, out=None, alpha=1.0, beta=0.0, transA=0, transB=0):
    """CUBLASMatmul2dFunc: alpha*op(A)*op(B) + beta*out."""
    A, B = _f32(A), _f32(B)
    M = A.shape[1] if transA else A.shape[0]
    Nn = B.shape[0] if transB else B.shape[1]
    o = np.zeros((M, Nn), np.float32) if out is None else _f32(out).copy()
    lib().occ_matmul2d(_fp(A), _dims(A.shape), _fp(B), _dims(B.shape), _fp(o),
                       C.c_float(alpha), C.c_float(beta), C.c_int64(transA), C.c_int64(transB))
    return o


def softmax(x, axis):
    x = _f32(x)
    y = np.empty_like(x)
    lib().occ_softmax(_fp(x), _fp(y), _dims(x.shape), C.c_int(x.ndim), C.c_int64(axis))
    return y
