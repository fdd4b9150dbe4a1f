"""ctypes front-end of ``liboccamy_replay.so``: builds the straight-line runtime-call
program an Occamy-compiled model would execute (lowering patterns, conv+bias+relu fusion,
liveness-placed deallocs, first-fit pool offsets -- see csrc/host/replay.cpp for the
reference files each step follows) and replays it against a library exporting the ABI.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import runtime

HERE = os.path.dirname(os.path.abspath(__file__))
REPLAY_PATH = os.path.join(HERE, "lib", "liboccamy_replay.so")

_i64p = C.POINTER(C.c_int64)
_lib = None

INSTR_NAMES = ("malloc", "dealloc", "h2d_const", "h2d_input", "d2h_output", "conv",
               "conv_bias_act", "tensor_op", "active", "clip", "maxpool", "avgpool", "reduce",
               "flatten", "matmul", "softmax")
POOL_NONE, POOL_FIRST_FIT, POOL_BY_SIZE = 0, 1, 2   # Program.lower(pool_opt=...)
FUSE_NONE, FUSE_REFERENCE, FUSE_WITH_CLIP = 0, 1, 2


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(REPLAY_PATH):
            raise RuntimeError(f"{REPLAY_PATH} is missing: run `python -m occamy_b200.build`")
        L = C.CDLL(REPLAY_PATH)
        L.occ_prog_create.restype = C.c_void_p
        L.occ_prog_destroy.argtypes = [C.c_void_p]
        L.occ_prog_error.restype = C.c_char_p
        L.occ_prog_error.argtypes = [C.c_void_p]
        L.occ_v_input.argtypes = [C.c_void_p, _i64p, C.c_int]
        L.occ_v_const.argtypes = [C.c_void_p, C.c_void_p, _i64p, C.c_int]
        L.occ_mark_output.argtypes = [C.c_void_p, C.c_int]
        L.occ_v_dims.argtypes = [C.c_void_p, C.c_int, _i64p, C.POINTER(C.c_int)]
        L.occ_op_conv.argtypes = [C.c_void_p] + [C.c_int] * 8
        L.occ_op_relu.argtypes = [C.c_void_p, C.c_int]
        L.occ_op_clip.argtypes = [C.c_void_p, C.c_int, C.c_float, C.c_float]
        L.occ_op_add.argtypes = [C.c_void_p, C.c_int, C.c_int]
        L.occ_op_maxpool.argtypes = [C.c_void_p] + [C.c_int] * 7
        L.occ_op_avgpool.argtypes = [C.c_void_p] + [C.c_int] * 7
        L.occ_op_gap.argtypes = [C.c_void_p, C.c_int]
        L.occ_op_flatten.argtypes = [C.c_void_p, C.c_int]
        L.occ_op_gemm.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_float,
                                  C.c_int, C.c_int]
        L.occ_op_softmax.argtypes = [C.c_void_p, C.c_int, C.c_int]
        L.occ_lower.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int64]
        L.occ_pool_bytes.restype = C.c_int64
        L.occ_pool_bytes.argtypes = [C.c_void_p]
        L.occ_lifetimes.restype = C.c_int
        L.occ_lifetimes.argtypes = [C.c_void_p, C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.c_int]
        L.occ_live_peak_bytes.restype = C.c_int64
        L.occ_live_peak_bytes.argtypes = [C.c_void_p]
        L.occ_sum_bytes.restype = C.c_int64
        L.occ_sum_bytes.argtypes = [C.c_void_p]
        L.occ_instr_counts.argtypes = [C.c_void_p, _i64p]
        L.occ_plan.argtypes = [C.c_void_p, _i64p, _i64p, C.c_int]
        L.occ_bind.restype = C.c_void_p
        L.occ_bind.argtypes = [C.c_char_p, C.c_char_p, C.c_int]
        L.occ_run.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.POINTER(C.c_void_p),
                              C.c_int]
        _lib = L
    return _lib


class Binding:
    """A shared library that exports the runtime ABI, bound for replay."""

    def __init__(self, so_path: str = runtime.LIB_PATH):
        err = C.create_string_buffer(512)
        self.handle = lib().occ_bind(so_path.encode(), err, 512)
        if not self.handle:
            raise RuntimeError(f"cannot bind {so_path}: {err.value.decode()}")
        self.path = so_path


class Program:
    """Graph builder + lowered program.  Value ids are plain ints."""

    def __init__(self):
        self.h = lib().occ_prog_create()
        self._keep = []      # constants: the program holds raw host pointers into these
        self.lowered = False

    def __del__(self):
        try:
            lib().occ_prog_destroy(self.h)
        except Exception:
            pass

    # ---- graph construction (ONNX-level operators, BN already folded) ----
    def input(self, shape):
        return lib().occ_v_input(self.h, runtime.dims(shape), len(shape))

    def const(self, array):
        a = np.ascontiguousarray(array, dtype=np.float32)
        self._keep.append(a)
        return lib().occ_v_const(self.h, a.ctypes.data, runtime.dims(a.shape), a.ndim)

    def conv(self, x, w, b=-1, groups=1, pads=(0, 0), strides=(1, 1)):
        return lib().occ_op_conv(self.h, x, w, b, groups, pads[0], pads[1], strides[0], strides[1])

    def relu(self, x):
        return lib().occ_op_relu(self.h, x)

    def clip(self, x, lo, hi):
        return lib().occ_op_clip(self.h, x, lo, hi)

    def add(self, a, b):
        return lib().occ_op_add(self.h, a, b)

    def maxpool(self, x, kernel, pads=(0, 0), strides=(1, 1)):
        return lib().occ_op_maxpool(self.h, x, kernel[0], kernel[1], pads[0], pads[1], strides[0],
                                    strides[1])

    def avgpool(self, x, kernel, pads=(0, 0), strides=(1, 1)):
        return lib().occ_op_avgpool(self.h, x, kernel[0], kernel[1], pads[0], pads[1], strides[0],
                                    strides[1])

    def gap(self, x):
        return lib().occ_op_gap(self.h, x)

    def flatten(self, x):
        return lib().occ_op_flatten(self.h, x)

    def gemm(self, a, b, c=-1, alpha=1.0, beta=1.0, transA=0, transB=0):
        return lib().occ_op_gemm(self.h, a, b, c, alpha, beta, transA, transB)

    def softmax(self, x, axis=1):
        return lib().occ_op_softmax(self.h, x, axis)

    def mark_output(self, v):
        lib().occ_mark_output(self.h, v)
        self._outputs = getattr(self, "_outputs", []) + [v]

    def shape(self, v):
        d = (C.c_int64 * 4)()
        r = C.c_int()
        lib().occ_v_dims(self.h, v, d, C.byref(r))
        return tuple(int(d[i]) for i in range(r.value))

    # ---- compiler back half ----
    def lower(self, fuse=FUSE_REFERENCE, dealloc_opt=True, pool_opt=True, workspace_bytes=0):
        n = lib().occ_lower(self.h, fuse, int(dealloc_opt), int(pool_opt), workspace_bytes)
        if n < 0:
            raise RuntimeError(lib().occ_prog_error(self.h).decode())
        self.lowered = True
        return n

    @property
    def pool_bytes(self):
        return int(lib().occ_pool_bytes(self.h))

    @property
    def live_peak_bytes(self):
        """Most bytes live at one point of the program: the lower bound of any pool plan."""
        return int(lib().occ_live_peak_bytes(self.h))

    @property
    def sum_bytes(self):
        return int(lib().occ_sum_bytes(self.h))

    def instr_counts(self):
        out = (C.c_int64 * 16)()
        lib().occ_instr_counts(self.h, out)
        return dict(zip(INSTR_NAMES, [int(v) for v in out]))

    def plan(self):
        n = lib().occ_plan(self.h, None, None, 0)
        off, by = (C.c_int64 * n)(), (C.c_int64 * n)()
        lib().occ_plan(self.h, off, by, n)
        return [(int(off[i]), int(by[i])) for i in range(n)]

    def lifetimes(self):
        """(malloc position, dealloc position) of every buffer, in the order of plan()."""
        n = lib().occ_lifetimes(self.h, None, None, 0)
        a, b = (C.c_int64 * n)(), (C.c_int64 * n)()
        lib().occ_lifetimes(self.h, a, b, n)
        return [(int(a[i]), int(b[i])) for i in range(n)]

    # ---- execution ----
    def run(self, binding: Binding, x: np.ndarray):
        """One inference from a host batch; returns the list of output arrays."""
        assert self.lowered
        x = np.ascontiguousarray(x, dtype=np.float32)
        outs = [np.empty(self.shape(v), np.float32) for v in self._outputs]
        ptrs = (C.c_void_p * len(outs))(*[o.ctypes.data for o in outs])
        rc = lib().occ_run(self.h, binding.handle, x.ctypes.data, 1, ptrs, 1)
        if rc:
            raise RuntimeError(f"occ_run failed: {rc}")
        return outs

    def run_raw(self, binding: Binding, input_ptr: int, input_kind: int, out_ptrs, copy_out: bool):
        """Replay with caller-managed memory: `input_ptr` is a host (kind 1) or device
        (kind 3) address; `out_ptrs` host addresses for the outputs."""
        ptrs = (C.c_void_p * max(1, len(out_ptrs)))(*out_ptrs)
        return lib().occ_run(self.h, binding.handle, input_ptr, input_kind, ptrs, int(copy_out))
