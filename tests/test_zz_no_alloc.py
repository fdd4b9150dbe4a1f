"""occamy_conv_bias_act_noalloc: the fused convolution for hosts that cannot allocate device
memory where they call the runtime (fixed start-up memory budgets, loops that must stay out
of the driver's allocator).  Its working copies live in a fixed array inside the library, so
the result must be the same as the allocating entry point's, call after call, although each
call finds the previous call's data in that array.

The file name sorts last on purpose: with `-x` every other test has run before this one.
"""
import ctypes as C

import numpy as np
import pytest

from occamy_b200 import runtime as rt
from oracle import ref

pytestmark = pytest.mark.gpu


def _conv_both(torch, x, w, b, pad, stride, act_mode):
    """Run the allocating entry point and the allocation-free one on the same device data;
    returns (reference result, allocation-free result, return code)."""
    L = rt.lib()
    N, Cc, H, W = x.shape
    K, _, R, S = w.shape
    P = (H + 2 * pad - R) // stride + 1
    Q = (W + 2 * pad - S) // stride + 1
    xd, wd, bd = (torch.from_numpy(a).cuda() for a in (x, w, b))
    y_ref_d = torch.zeros((N, K, P, Q), dtype=torch.float32, device="cuda")
    y_new_d = torch.full((N, K, P, Q), float("nan"), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()

    # existing entry point (bf16 tensor-core mode), read back through the ABI's own copy
    rt.set_math_mode(rt.MATH_BF16)
    h = C.c_void_p()
    L.cudnnCreate(C.byref(h))
    L.DNNConvBiasActivFunc(h, xd.data_ptr(), rt.dims(x.shape), wd.data_ptr(), rt.dims(w.shape),
                           bd.data_ptr(), rt.dims((1, K, 1, 1)), None, 0, 1, rt.dims((pad, pad)),
                           rt.dims((stride, stride)), act_mode, y_ref_d.data_ptr())
    y_ref = np.empty((N, K, P, Q), np.float32)
    L.wrapDNNMemcpy(y_ref.ctypes.data, y_ref_d.data_ptr(), y_ref.nbytes, 2, None)
    L.cudnnDestroy(h)
    rt.synchronize()

    # allocation-free entry point on the legacy default stream
    rc = L.occamy_conv_bias_act_noalloc(xd.data_ptr(), rt.dims(x.shape), wd.data_ptr(),
                                        rt.dims(w.shape), bd.data_ptr(), rt.dims((pad, pad)),
                                        rt.dims((stride, stride)), act_mode, y_new_d.data_ptr(),
                                        None)
    torch.cuda.synchronize()
    return y_ref, y_new_d.cpu().numpy(), rc


def test_noalloc_matches_allocating_entry_point_twice_in_a_row(native_libs):
    torch = pytest.importorskip("torch")
    rt.last_error(clear=True)
    r = np.random.Generator(np.random.PCG64(77))
    # two different problems back to back: the second call finds the first one's data in
    # the shared array and must not be affected by it
    cases = [((1, 64, 56, 56), (64, 64, 3, 3), 1, 1, 1), ((2, 32, 20, 20), (48, 32, 1, 1), 0, 2, 5)]
    for xs, ws, pad, stride, act in cases:
        x = r.uniform(-1, 1, xs).astype(np.float32)
        w = r.normal(0, np.sqrt(2.0 / (ws[1] * ws[2] * ws[3])), ws).astype(np.float32)
        b = r.normal(0, 0.1, ws[0]).astype(np.float32)
        y_ref, y_new, rc = _conv_both(torch, x, w, b, pad, stride, act)
        assert rc == 0
        assert np.isfinite(y_new).all()
        scale = np.abs(y_ref).max()
        # same kernel, same operands: the tolerance of the bf16 tests is far from needed
        assert np.abs(y_new - y_ref).max() <= 2e-2 * scale
        assert np.array_equal(y_new, y_ref)
        # and against the CPU oracle, within the tensor-core mode's bound
        want = ref.conv2d(x, w, b, (pad, pad), (stride, stride), act=act)
        assert np.abs(y_new - want).max() <= 2e-2 * np.abs(want).max()
    assert rt.lib().occamy_noalloc_last_error(0) == 0
    assert rt.last_error(clear=True) == 0


def test_noalloc_leaves_free_device_memory_unchanged(native_libs):
    """The point of the entry point: a call takes no device memory.  The first call on a device
    is left out of the comparison (the driver loads the kernels' code then); from the second
    call on, free memory as the driver reports it is the same before and after."""
    torch = pytest.importorskip("torch")
    L = rt.lib()
    r = np.random.Generator(np.random.PCG64(78))
    x = torch.from_numpy(r.uniform(-1, 1, (2, 64, 28, 28)).astype(np.float32)).cuda()
    w = torch.from_numpy(r.normal(0, 0.05, (128, 64, 3, 3)).astype(np.float32)).cuda()
    b = torch.zeros(128, device="cuda")
    y = torch.empty((2, 128, 28, 28), device="cuda")

    def call():
        rc = L.occamy_conv_bias_act_noalloc(x.data_ptr(), rt.dims(x.shape), w.data_ptr(),
                                            rt.dims(w.shape), b.data_ptr(), rt.dims((1, 1)),
                                            rt.dims((1, 1)), 1, y.data_ptr(), None)
        torch.cuda.synchronize()
        return rc

    assert call() == 0
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        assert call() == 0
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0
    assert L.occamy_noalloc_last_error(1) == 0
    assert 0 < L.occamy_noalloc_capacity() < 32 << 20


def test_noalloc_rejects_what_does_not_fit(native_libs):
    torch = pytest.importorskip("torch")
    L = rt.lib()
    # 64 x 64 x 112 x 112 needs ~ 3 x 100 MB of working copies: over the fixed 32 MiB.
    # Only shapes are inspected before the refusal, so tiny dummy buffers are enough.
    d = torch.zeros(16, device="cuda")
    rc = L.occamy_conv_bias_act_noalloc(d.data_ptr(), rt.dims((64, 64, 112, 112)), d.data_ptr(),
                                        rt.dims((64, 64, 3, 3)), d.data_ptr(), rt.dims((1, 1)),
                                        rt.dims((1, 1)), 1, d.data_ptr(), None)
    assert rc == -2
    rc = L.occamy_conv_bias_act_noalloc(d.data_ptr(), rt.dims((1, 20, 8, 8)), d.data_ptr(),
                                        rt.dims((8, 20, 3, 3)), d.data_ptr(), rt.dims((1, 1)),
                                        rt.dims((1, 1)), 1, d.data_ptr(), None)
    assert rc == -3
    # extents beyond INT_MAX, a negative pad, a filter larger than the padded image
    for dx, dw, pads in ((((1 << 33), 16, 8, 8), (16, 16, 3, 3), (1, 1)),
                         ((1, 16, 8, 8), (16, 16, 3, 3), (-1, 0)),
                         ((1, 16, 2, 2), (16, 16, 5, 5), (1, 1))):
        rc = L.occamy_conv_bias_act_noalloc(d.data_ptr(), rt.dims(dx), d.data_ptr(), rt.dims(dw),
                                            d.data_ptr(), rt.dims(pads), rt.dims((2, 2)), 1,
                                            d.data_ptr(), None)
        assert rc == -3, (dx, dw, pads)
    torch.cuda.synchronize()
