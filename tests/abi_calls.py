"""Thin test-side wrappers that call single runtime symbols through the C ABI with host
numpy data: upload with wrapDNNMemcpy, call, download.  They keep tensors on the device
between calls when asked, so chains of calls exercise the runtime's internal formats."""
import ctypes as C

import numpy as np

from occamy_b200 import runtime as rt


class Dev:
    """A device tensor with its logical shape."""

    def __init__(self, shape, data=None):
        self.shape = tuple(int(s) for s in shape)
        n = int(np.prod(self.shape)) if len(self.shape) else 1
        if data is not None:
            self.buf = rt.DeviceBuffer.from_numpy(np.ascontiguousarray(data, np.float32))
        else:
            self.buf = rt.DeviceBuffer(max(n, 1) * 4)
        self.ptr = self.buf.ptr

    def numpy(self):
        return self.buf.to_numpy(self.shape)


def up(a):
    return Dev(a.shape, a)


_handle = None


def handle():
    global _handle
    if _handle is None:
        h = C.c_void_p()
        rt.lib().cudnnCreate(C.byref(h))
        _handle = h
    return _handle


def conv(x: Dev, w: Dev, bias=None, pads=(0, 0), strides=(1, 1), groups=1, act_mode=None):
    """DNNConvFunc (act_mode None; bias ignored) or DNNConvBiasActivFunc (act_mode 1/3/5)."""
    N, Cc, H, W = x.shape
    K, _, R, S = w.shape
    P = (H + 2 * pads[0] - R) // strides[0] + 1
    Q = (W + 2 * pads[1] - S) // strides[1] + 1
    y = Dev((N, K, P, Q))
    L = rt.lib()
    if act_mode is None:
        r = L.DNNConvFunc(handle(), x.ptr, rt.dims(x.shape), w.ptr, rt.dims(w.shape), None, 0, 1,
                          groups, rt.dims(pads), rt.dims(strides), y.ptr)
    else:
        r = L.DNNConvBiasActivFunc(handle(), x.ptr, rt.dims(x.shape), w.ptr, rt.dims(w.shape),
                                   bias.ptr, rt.dims((1, K, 1, 1)), None, 0, 1, rt.dims(pads),
                                   rt.dims(strides), act_mode, y.ptr)
    assert r == y.ptr, "compute entry points return the output pointer"
    return y


def tensor_op(mode, A: Dev, B: Dev, out: Dev = None, bias=1.0):
    out = out or Dev(A.shape)
    r = rt.lib().DNNTensorOpFunc(handle(), mode, A.ptr, rt.dims(A.shape), len(A.shape), B.ptr,
                                 rt.dims(B.shape), len(B.shape), out.ptr, rt.dims(A.shape),
                                 len(A.shape), bias)
    assert r == out.ptr
    return out


def active(x: Dev, mode=1):
    y = Dev(x.shape)
    d = list(x.shape) + [1] * (4 - len(x.shape))
    assert rt.lib().DNNActiveFunc(handle(), x.ptr, rt.dims(d), mode, y.ptr) == y.ptr
    return y


def clip(x: Dev, lo, hi):
    y = Dev(x.shape)
    assert rt.lib().CUDAClipFunc(x.ptr, y.ptr, rt.dims(x.shape), lo, hi, len(x.shape)) == y.ptr
    return y


def pool(x: Dev, kernel, pads=(0, 0), strides=(1, 1), avg=False):
    N, Cc, H, W = x.shape
    P = (H + 2 * pads[0] - kernel[0]) // strides[0] + 1
    Q = (W + 2 * pads[1] - kernel[1]) // strides[1] + 1
    y = Dev((N, Cc, P, Q))
    fn = rt.lib().DNNAveragePoolFunc if avg else rt.lib().DNNMaxPoolFunc
    # ONNX pad order (h_begin, w_begin, h_end, w_end); the runtime reads [0] and [2]
    r = fn(handle(), x.ptr, rt.dims(x.shape), y.ptr, rt.dims(y.shape), rt.dims(kernel),
           rt.dims((pads[0], pads[1], pads[1], pads[1])), rt.dims(strides))
    assert r == y.ptr
    return y


def reduce_mean(x: Dev, out_shape):
    y = Dev(out_shape)
    r = rt.lib().DNNReduceFunc(handle(), len(x.shape), x.ptr, rt.dims(x.shape), y.ptr,
                               rt.dims(out_shape), 5)
    assert r == y.ptr
    return y


def matmul2d(A: Dev, B: Dev, alpha=1.0, beta=0.0, transA=0, transB=0, out: Dev = None):
    M = A.shape[1] if transA else A.shape[0]
    Nn = B.shape[0] if transB else B.shape[1]
    out = out or Dev((M, Nn))
    r = rt.lib().CUBLASMatmul2dFunc(2, A.ptr, rt.dims(A.shape), B.ptr, rt.dims(B.shape), out.ptr,
                                    rt.dims(out.shape), out.ptr, rt.dims(out.shape), alpha, beta,
                                    transA, transB)
    assert r == out.ptr
    return out


def softmax(x: Dev, axis):
    y = Dev(x.shape)
    r = rt.lib().CUDASoftmaxFunc(x.ptr, rt.dims(x.shape), y.ptr, rt.dims(x.shape), axis,
                                 len(x.shape))
    assert r == y.ptr
    return y


def flatten(x: Dev):
    y = Dev((x.shape[0], int(np.prod(x.shape[1:]))))
    r = rt.lib().CUDAFlattenFunc(x.ptr, rt.dims(x.shape), y.ptr, rt.dims(y.shape), 1, len(x.shape))
    assert r == y.ptr
    return y


def reshape(x: Dev, new_shape):
    y = Dev(new_shape)
    r = rt.lib().CUDAReshapeFunc(x.ptr, rt.dims(x.shape), len(x.shape), y.ptr)
    assert r == y.ptr
    return y
