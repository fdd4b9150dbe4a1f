"""The runtime symbols outside the CNN graphs (transposes, concat, gather, expand, squeeze,
cast, unary maps, non-zero, N-d matmul), each called through the C ABI on a B200 and compared
with numpy on the same seeded data.  Integer and index results must be bit-exact, float maps
within 1e-6 relative (1e-5 for the transcendental ones).

The quirks of the reference's definitions are part of the contract and are tested as such:
the cast returns its INPUT pointer (cuda/CUDACastI64toFloatFunc.cu:12), PRelu reads slope[0]
only (cuda/CUDAPReluFunc.cu:17), Pow takes one scalar exponent from device memory
(cuda/CUDAPowFunc.cu:16), Expand / Squeeze / Unsqueeze are plain copies, NonZero writes the
flat indices of the non-zero elements in order (cuda/CUDANonZeroFloatFunc.cu:19-29).
"""
import ctypes as C

import numpy as np
import pytest

from helpers import max_rel_err
from occamy_b200 import runtime as rt

pytestmark = pytest.mark.gpu

_i64p = C.POINTER(C.c_int64)


@pytest.fixture(autouse=True)
def _check_runtime_errors(native_libs):
    rt.last_error(clear=True)
    yield
    rt.synchronize()
    assert rt.last_error(clear=True) == 0


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def dev(a):
    return rt.DeviceBuffer.from_numpy(np.ascontiguousarray(a))


def empty(shape, dtype):
    n = int(np.prod(shape)) if len(shape) else 1
    return rt.DeviceBuffer(max(n, 1) * np.dtype(dtype).itemsize)


PERMS = {2: [(1, 0), (0, 1)], 3: [(2, 0, 1), (0, 2, 1), (1, 0, 2)],
         4: [(0, 2, 3, 1), (0, 3, 1, 2), (3, 2, 1, 0), (1, 0, 2, 3)],
         6: [(0, 1, 4, 2, 5, 3), (5, 4, 3, 2, 1, 0)]}
SHAPES = {2: (37, 65), 3: (5, 33, 17), 4: (2, 24, 9, 7), 6: (2, 3, 4, 2, 5, 3)}


@pytest.mark.parametrize("rank", [2, 3, 4, 6])
@pytest.mark.parametrize("kind", ["Float", "Int64"])
def test_transpose(rank, kind):
    dtype = np.float32 if kind == "Float" else np.int64
    shape = SHAPES[rank]
    x = (rng(rank).normal(0, 1, shape) * 100).astype(dtype)
    fn = getattr(rt.lib(), f"CUDATranspose{rank}D{kind}Func")
    for perm in PERMS[rank]:
        want = np.transpose(x, perm)
        xd, yd = dev(x), empty(want.shape, dtype)
        r = fn(xd.ptr, rt.dims(shape), yd.ptr, rt.dims(want.shape), rt.dims(perm), rank)
        assert r == yd.ptr
        assert np.array_equal(yd.to_numpy(want.shape, dtype), want)


@pytest.mark.parametrize("kind", ["Float", "Int64"])
@pytest.mark.parametrize("case", [((2, 3, 4), (2, 5, 4), (2, 1, 4), 1), ((3, 4), (3, 6), None, -1),
                                  ((2, 2, 3, 3), (1, 2, 3, 3), None, 0)])
def test_concat(kind, case):
    dtype = np.float32 if kind == "Float" else np.int64
    *shapes, axis = case
    shapes = [s for s in shapes if s is not None]
    r = rng(21)
    xs = [(r.normal(0, 1, s) * 50).astype(dtype) for s in shapes]
    want = np.concatenate(xs, axis=axis)
    bufs = [dev(x) for x in xs]
    ptrs = (C.c_void_p * len(xs))(*[b.ptr for b in bufs])
    dim_arrays = [rt.dims(s) for s in shapes]
    dim_list = (_i64p * len(xs))(*[C.cast(d, _i64p) for d in dim_arrays])
    out = empty(want.shape, dtype)
    fn = getattr(rt.lib(), f"CUDAConcat{kind}Func")
    ret = fn(ptrs, dim_list, out.ptr, rt.dims(want.shape), axis, len(xs), len(shapes[0]))
    assert ret == out.ptr
    assert np.array_equal(out.to_numpy(want.shape, dtype), want)


@pytest.mark.parametrize("kind", ["Float", "Int64"])
@pytest.mark.parametrize("case", [((5, 7), (3,), 0), ((5, 7), (2, 2), 1), ((2, 6, 3), (4,), 1),
                                  ((4, 3), (1,), -1)])
def test_gather(kind, case):
    dtype = np.float32 if kind == "Float" else np.int64
    shape, idx_shape, axis = case
    r = rng(22)
    x = (r.normal(0, 1, shape) * 50).astype(dtype)
    ax = axis % len(shape)
    idx = r.integers(-shape[ax], shape[ax], idx_shape).astype(np.int64)   # negative indices wrap
    want = np.take(x, idx, axis=axis)
    xd, idd, out = dev(x), dev(idx), empty(want.shape, dtype)
    fn = getattr(rt.lib(), f"CUDAGather{kind}Func")
    ret = fn(xd.ptr, rt.dims(shape), len(shape), out.ptr, rt.dims(want.shape), want.ndim, idd.ptr,
             rt.dims(idx_shape), len(idx_shape), axis)
    assert ret == out.ptr
    assert np.array_equal(out.to_numpy(want.shape, dtype), want)


def test_expand_squeeze_unsqueeze_are_copies():
    L = rt.lib()
    r = rng(23)
    xi = r.integers(-1000, 1000, (3, 1, 5)).astype(np.int64)
    xf = r.normal(0, 1, (3, 1, 5)).astype(np.float32)
    xid, xfd = dev(xi), dev(xf)
    out = empty(xi.shape, np.int64)
    shape_d = dev(np.array(xi.shape, np.int64))
    assert L.CUDAExpandInt64Func(xid.ptr, rt.dims(xi.shape), 3, out.ptr, rt.dims(xi.shape),
                                 shape_d.ptr, rt.dims((3,))) == out.ptr
    assert np.array_equal(out.to_numpy(xi.shape, np.int64), xi)
    for name, x, xd, dtype in (("Float", xf, xfd, np.float32), ("Int64", xi, xid, np.int64)):
        for op, oshape in (("Squeeze", (3, 5)), ("Unsqueeze", (3, 1, 1, 5))):
            o = empty(oshape, dtype)
            fn = getattr(L, f"CUDA{op}{name}Func")
            assert fn(xd.ptr, rt.dims(x.shape), o.ptr, rt.dims(oshape), 1, 3) == o.ptr
            assert np.array_equal(o.to_numpy(oshape, dtype), x.reshape(oshape))


def test_cast_returns_its_input_pointer():
    x = rng(24).integers(-2**40, 2**40, (4, 9)).astype(np.int64)
    xd, out = dev(x), empty(x.shape, np.float32)
    ret = rt.lib().CUDACastI64toFloatFunc(xd.ptr, out.ptr, rt.dims(x.shape), 2)
    assert ret == xd.ptr          # the reference returns the input, and callers may rely on it
    assert np.array_equal(out.to_numpy(x.shape), x.astype(np.float32))


def test_unary_maps():
    L = rt.lib()
    x = rng(25).normal(0, 2, (3, 5, 7)).astype(np.float32)
    x[0, 0, 0] = 0.0
    xd = dev(x)
    d, rank = rt.dims(x.shape), 3

    def run(fn, *args):
        out = empty(x.shape, np.float32)
        assert fn(*[out.ptr if a is Ellipsis else a for a in args]) == out.ptr
        return out.to_numpy(x.shape)

    from math import erf
    want_erf = np.vectorize(erf)(x.astype(np.float64))
    assert max_rel_err(run(L.CUDAErfFunc, xd.ptr, ..., d, rank), want_erf) <= 1e-5
    assert max_rel_err(run(L.CUDALeakyReluFunc, xd.ptr, ..., d, 0.1, rank),
                       np.where(x >= 0, x, np.float32(0.1) * x)) <= 1e-6
    assert np.array_equal(run(L.CUDANegativeFunc, xd.ptr, ..., d, rank), -x)
    nz = np.where(x == 0, np.float32(1), x)
    nzd = dev(nz)
    assert max_rel_err(run(L.CUDAReciprocalFunc, nzd.ptr, ..., d, rank), 1.0 / nz) <= 1e-6
    # PRelu: slope[0] only, whatever else the slope tensor holds
    slope = dev(np.array([0.25, 99.0, -7.0], np.float32))
    assert max_rel_err(run(L.CUDAPReluFunc, xd.ptr, ..., d, slope.ptr, rank),
                       np.where(x >= 0, x, np.float32(0.25) * x)) <= 1e-6
    # Pow: one scalar exponent read from device memory
    pos = np.abs(x) + np.float32(0.5)
    posd, expo = dev(pos), dev(np.array([1.5], np.float32))
    out = empty(x.shape, np.float32)
    assert L.CUDAPowFunc(posd.ptr, expo.ptr, out.ptr, d, rank) == out.ptr
    assert max_rel_err(out.to_numpy(x.shape), pos.astype(np.float64) ** 1.5) <= 1e-5


@pytest.mark.parametrize("kind", ["Float", "Int64"])
@pytest.mark.parametrize("n", [1, 31, 1024, 5000])
def test_nonzero(kind, n):
    dtype = np.float32 if kind == "Float" else np.int64
    r = rng(26 + n)
    x = (r.integers(0, 3, (n,)) * r.integers(0, 2, (n,))).astype(dtype)
    want = np.flatnonzero(x).astype(dtype)
    xd, out = dev(x), empty((n,), dtype)     # fresh buffers read as zero past the last index
    fn = getattr(rt.lib(), f"CUDANonZero{kind}Func")
    assert fn(xd.ptr, rt.dims((n,)), out.ptr, rt.dims((n,)), 1) == out.ptr
    got = out.to_numpy((n,), dtype)
    assert np.array_equal(got[:len(want)], want)
    assert not got[len(want):].any()


@pytest.mark.parametrize("case", [((3, 4, 5), (3, 5, 6)), ((2, 3, 4, 5), (5, 7)), ((2, 3, 4, 5), (3, 5, 2)),
                                  ((6, 8), (8, 3)), ((4, 64, 96), (96, 80)), ((7, 5), (2, 5, 3))])
def test_matmul_nd(case):
    sa, sb = case
    r = rng(27)
    a = r.normal(0, 1, sa).astype(np.float32)
    b = r.normal(0, 1, sb).astype(np.float32)
    want = np.matmul(a.astype(np.float64), b.astype(np.float64))
    ad, bd, out = dev(a), dev(b), empty(want.shape, np.float32)
    ret = rt.lib().CUDAMatmulNdFunc(ad.ptr, rt.dims(sa), len(sa), bd.ptr, rt.dims(sb), len(sb),
                                    out.ptr, rt.dims(want.shape), want.ndim)
    assert ret == out.ptr
    assert max_rel_err(out.to_numpy(want.shape), want) <= 1e-5
