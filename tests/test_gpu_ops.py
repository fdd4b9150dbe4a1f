"""Parity of every hot-path runtime symbol, called through the C ABI on a B200, against
the CPU oracle on the same seeded inputs.

Tolerances (per tensor, max|y - ref| / max|ref|):
  fp32 mode                                <= 1e-4
  bf16 and fp16 tensor-core modes          <= 2e-2
"""
import numpy as np
import pytest

import abi_calls as A
from helpers import max_rel_err
from occamy_b200 import runtime as rt
from oracle import ref

pytestmark = pytest.mark.gpu

# fp32 mode runs dense convolutions and GEMMs on the tensor cores (operands split into bf16
# parts); FP32_CUDA_CORES is the same mode with that switched off, so that the CUDA-core kernels
# stay covered.
FP32_CUDA_CORES = -1
TOL = {rt.MATH_FP32: 1e-4, FP32_CUDA_CORES: 1e-4, rt.MATH_BF16: 2e-2, rt.MATH_F16: 2e-2}
MODES = [rt.MATH_FP32, FP32_CUDA_CORES, rt.MATH_BF16, rt.MATH_F16]


def set_mode(mode):
    rt.lib().occamy_set_fp32_tensor_cores(0 if mode == FP32_CUDA_CORES else 1)
    rt.set_math_mode(rt.MATH_FP32 if mode == FP32_CUDA_CORES else mode)
# output rounding of the 16-bit formats (one step of the stored value, relative)
STEP = {rt.MATH_BF16: 2.0 ** -8, rt.MATH_F16: 2.0 ** -11}


@pytest.fixture(autouse=True)
def _check_runtime_errors(native_libs):
    rt.last_error(clear=True)
    yield
    rt.synchronize()
    rt.lib().occamy_set_fp32_tensor_cores(1)
    assert rt.last_error(clear=True) == 0


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def he(r, K, C, R, S):
    return r.normal(0, np.sqrt(2.0 / (C * R * S)), (K, C, R, S)).astype(np.float32)


# (N, C, H, W, K, R, pad, stride, groups)
CONV_CASES = [
    (1, 64, 56, 56, 64, 3, 1, 1, 1),      # the single-conv benchmark configuration
    (2, 64, 28, 28, 256, 1, 0, 1, 1),     # 1x1: flat GEMM view
    (2, 256, 28, 28, 128, 1, 0, 2, 1),    # 1x1 stride 2 (ResNet v1 down-sampling)
    (2, 128, 28, 28, 128, 3, 1, 2, 1),    # 3x3 stride 2 (v1.5): four stride phases
    (3, 512, 7, 7, 512, 3, 1, 1, 1),      # 7x7 maps: several images per tile
    (2, 3, 64, 64, 64, 7, 3, 2, 1),       # RGB stem: width taps folded into channels
    (2, 3, 32, 32, 64, 3, 1, 1, 1),       # VGG first layer
    (1, 32, 13, 11, 24, 3, 1, 1, 1),      # ragged: K < tile, odd H/W, 32-channel K block
    (2, 16, 9, 9, 40, 1, 0, 1, 1),        # 16-channel K block
    (1, 48, 10, 10, 96, 3, 1, 1, 1),      # 48 = 3 x 16-channel blocks
    (1, 320, 7, 7, 1280, 1, 0, 1, 1),     # MobileNetV2 head; K = 5 x 256
    (2, 24, 14, 14, 144, 1, 0, 1, 1),     # 24 input channels: zero-padded to 32 for the MMA
    (1, 40, 9, 9, 24, 3, 1, 1, 1),        # 40 -> 48 padded, 3x3 with halo
    (2, 8, 12, 12, 8, 3, 1, 1, 2),        # grouped (CUDA-core path in both modes)
    (2, 20, 9, 9, 10, 3, 0, 1, 1),        # channel counts no tensor-core tile fits
    (2, 32, 16, 16, 32, 3, 1, 1, 32),     # depthwise stride 1
    (2, 96, 15, 15, 96, 3, 1, 2, 96),     # depthwise stride 2, odd size
    (1, 64, 5, 5, 64, 5, 2, 1, 1),        # 5x5: 25 taps
]


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("case", CONV_CASES)
@pytest.mark.parametrize("act_mode", [None, 1, 5, 3])
def test_conv(case, mode, act_mode):
    N, C, H, W, K, R, pad, stride, groups = case
    if act_mode is not None and groups != 1:
        pytest.skip("the fused symbol has no group argument")
    r = rng(hash(case) % 2**31)
    x = r.uniform(-1, 1, (N, C, H, W)).astype(np.float32)
    w = he(r, K, C // groups, R, R)
    b = r.normal(0, 0.5, K).astype(np.float32)
    set_mode(mode)
    y = A.conv(A.up(x), A.up(w), A.up(b) if act_mode is not None else None, (pad, pad),
               (stride, stride), groups, act_mode).numpy()
    lo, hi = (0.0, 6.0) if act_mode == 3 else (0.0, 0.0)
    want = ref.conv2d(x, w, b if act_mode is not None else None, (pad, pad), (stride, stride),
                      groups, act=act_mode if act_mode is not None else 5, lo=lo, hi=hi)
    assert y.shape == want.shape
    assert max_rel_err(y, want) <= TOL[mode]


@pytest.mark.parametrize("mode", MODES)
def test_conv_empty_and_tiny(mode):
    set_mode(mode)
    r = rng(5)
    # batch 0: nothing to do, pointer still returned
    x0 = A.Dev((0, 16, 4, 4))
    w = A.up(he(r, 16, 16, 1, 1))
    y0 = A.conv(x0, w)
    assert y0.shape == (0, 16, 4, 4)
    # 1x1 spatial
    x = r.uniform(-1, 1, (1, 16, 1, 1)).astype(np.float32)
    y = A.conv(A.up(x), w).numpy()
    assert max_rel_err(y, ref.conv2d(x, w.numpy())) <= TOL[mode]


@pytest.mark.parametrize("mode", MODES)
def test_unfused_chain_matches_fused(mode):
    """conv -> in-place bias add -> relu (what the compiler emits without fusion), then
    residual add, max pool and global average pool on the same device tensors."""
    set_mode(mode)
    r = rng(11)
    x = r.uniform(-1, 1, (2, 64, 14, 14)).astype(np.float32)
    w = he(r, 64, 64, 3, 3)
    b = r.normal(0, 0.1, 64).astype(np.float32)
    xd, wd, bd = A.up(x), A.up(w), A.up(b)
    y = A.conv(xd, wd, pads=(1, 1))
    y = A.tensor_op(0, y, A.Dev((1, 64, 1, 1), b), out=y)          # in place
    y = A.active(y, 1)
    fused = A.conv(xd, wd, bd, pads=(1, 1), act_mode=1)
    want = ref.conv2d(x, w, b, (1, 1), (1, 1), act=1)
    assert max_rel_err(y.numpy(), want) <= TOL[mode]
    assert max_rel_err(fused.numpy(), want) <= TOL[mode]
    s = A.tensor_op(0, y, fused)                                    # residual-style add
    want_s = want + want
    assert max_rel_err(s.numpy(), want_s) <= TOL[mode]
    p = A.pool(s, (3, 3), (1, 1), (2, 2))
    want_p = ref.pool2d(want_s, (3, 3), (1, 1), (2, 2))
    assert max_rel_err(p.numpy(), want_p) <= TOL[mode]
    g = A.reduce_mean(p, (2, 64, 1, 1))
    assert max_rel_err(g.numpy(), ref.reduce_mean(want_p, (2, 64, 1, 1))) <= TOL[mode]
    c = A.clip(s, 0.5, 1.5)
    assert max_rel_err(c.numpy(), ref.clip(want_s, 0.5, 1.5)) <= TOL[mode]
    f = A.flatten(p)
    assert max_rel_err(f.numpy(), want_p.reshape(2, -1)) <= TOL[mode]


@pytest.mark.parametrize("shapes", [((2, 8, 5, 7), (2, 8, 5, 7)), ((2, 8, 5, 7), (1, 8, 1, 1)),
                                    ((4, 10), (1, 10)), ((3, 4, 5, 6), (1, 1, 5, 6)),
                                    ((2, 3, 4, 5), (2, 3, 1, 1))])
@pytest.mark.parametrize("op", [0, 1])
def test_tensor_op_broadcast(shapes, op):
    rt.set_math_mode(rt.MATH_FP32)
    r = rng(3)
    a = r.normal(0, 1, shapes[0]).astype(np.float32)
    b = r.normal(0, 1, shapes[1]).astype(np.float32)
    y = A.tensor_op(op, A.up(a), A.up(b), bias=0.5).numpy()
    assert max_rel_err(y, ref.tensor_op(op, a, b, 0.5)) <= 1e-6


def test_tensor_op_sqrt():
    rt.set_math_mode(rt.MATH_FP32)
    a = rng(4).uniform(0, 4, (2, 3, 5, 5)).astype(np.float32)
    y = A.tensor_op(4, A.up(a), A.up(a)).numpy()
    assert max_rel_err(y, np.sqrt(a)) <= 1e-6


@pytest.mark.parametrize("mode_act", [0, 1, 2])
def test_activation(mode_act):
    rt.set_math_mode(rt.MATH_FP32)
    x = rng(6).normal(0, 2, (2, 5, 7, 3)).astype(np.float32)
    y = A.active(A.up(x), mode_act).numpy()
    assert max_rel_err(y, ref.activation(x, mode_act)) <= 1e-5


@pytest.mark.parametrize("case", [((2, 64, 112, 112), (3, 3), (1, 1), (2, 2)),
                                  ((2, 16, 8, 8), (2, 2), (0, 0), (2, 2)),
                                  ((1, 5, 9, 7), (3, 3), (1, 1), (1, 1)),
                                  ((1, 8, 7, 7), (7, 7), (0, 0), (1, 1)),
                                  ((2, 8, 6, 6), (1, 1), (0, 0), (1, 1))])
@pytest.mark.parametrize("avg", [False, True])
def test_pool(case, avg):
    rt.set_math_mode(rt.MATH_FP32)
    shape, k, p, s = case
    x = rng(7).normal(0, 1, shape).astype(np.float32)
    y = A.pool(A.up(x), k, p, s, avg).numpy()
    want = ref.pool2d(x, k, p, s, avg=avg, count_include_pad=True)
    assert max_rel_err(y, want) <= 1e-6


@pytest.mark.parametrize("shapes", [((4, 32, 7, 7), (4, 32, 1, 1)), ((3, 5, 4, 6), (3, 1, 4, 1)),
                                    ((6, 10), (6, 1)), ((2, 3, 4, 5), (1, 1, 1, 1))])
def test_reduce_mean(shapes):
    rt.set_math_mode(rt.MATH_FP32)
    x = rng(8).normal(0, 1, shapes[0]).astype(np.float32)
    y = A.reduce_mean(A.up(x), shapes[1]).numpy()
    assert max_rel_err(y, ref.reduce_mean(x, shapes[1])) <= 1e-5


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("case", [(256, 2048, 1000, 0, 1), (4, 64, 10, 0, 1), (3, 20, 7, 0, 0),
                                  (5, 16, 9, 1, 0), (64, 512, 96, 0, 1), (1, 2048, 1000, 0, 1)])
def test_matmul2d(case, mode):
    M, K, Nn, tA, tB = case
    set_mode(mode)
    r = rng(9)
    a = r.normal(0, 1, (K, M) if tA else (M, K)).astype(np.float32)
    b = (r.normal(0, 1, (Nn, K) if tB else (K, Nn)) / np.sqrt(K)).astype(np.float32)
    y = A.matmul2d(A.up(a), A.up(b), 1.0, 1.0, tA, tB).numpy()   # beta = 1 on a zeroed output
    want = ref.matmul2d(a, b, None, 1.0, 0.0, tA, tB)
    assert max_rel_err(y, want) <= TOL[mode]


def test_matmul2d_alpha_beta_accumulates():
    rt.set_math_mode(rt.MATH_FP32)
    r = rng(10)
    a = r.normal(0, 1, (6, 12)).astype(np.float32)
    b = r.normal(0, 1, (12, 5)).astype(np.float32)
    c = r.normal(0, 1, (6, 5)).astype(np.float32)
    out = A.up(c)
    y = A.matmul2d(A.up(a), A.up(b), 0.5, 2.0, 0, 0, out=out).numpy()
    assert max_rel_err(y, 0.5 * (a @ b) + 2.0 * c) <= 1e-5


@pytest.mark.parametrize("shape_axis", [((256, 1000), 1), ((3, 7), 1), ((2, 5, 4, 3), 1),
                                        ((4, 6), 0), ((2, 3, 8), 2)])
def test_softmax(shape_axis):
    shape, axis = shape_axis
    x = rng(12).normal(0, 3, shape).astype(np.float32)
    y = A.softmax(A.up(x), axis).numpy()
    want = ref.softmax(x, axis)
    assert max_rel_err(y, want) <= 1e-5
    # index outputs are bit-exact
    assert np.array_equal(y.argmax(axis), want.argmax(axis))


def test_zero_fill_contract():
    """A tensor handed out by the allocator reads as zero until written (the reference
    memsets on every malloc / mem-offset)."""
    d = A.Dev((3, 4, 5, 6))
    assert not d.numpy().any()
    # max pool of an untouched (zero) tensor, then an op that accumulates into its output
    p = A.pool(d, (2, 2), (0, 0), (1, 1))
    assert not p.numpy().any()


def test_pool_offsets_and_reuse():
    """wrapDNNMemPoolInit + wrapDNNMemOffset: tensors live at base + offset; a range that is
    handed out again reads as zero again."""
    import ctypes as C
    L = rt.lib()
    base = C.c_void_p()
    L.wrapDNNMemPoolInit(C.byref(base), 1 << 20)
    p1, p2 = C.c_void_p(), C.c_void_p()
    L.wrapDNNMemOffset(C.byref(p1), base, 4096, 4000)
    assert p1.value == base.value + 4096
    data = np.arange(1000, dtype=np.float32)
    L.wrapDNNMemcpy(p1, data.ctypes.data, 4000, 1, None)
    back = np.empty(1000, np.float32)
    L.wrapDNNMemcpy(back.ctypes.data, p1, 4000, 2, None)
    assert np.array_equal(back, data)
    L.wrapDNNMemOffset(C.byref(p2), base, 4096 + 2000, 4000)   # overlaps the first tensor
    L.wrapDNNMemcpy(back.ctypes.data, p2, 4000, 2, None)
    assert not back.any()
    L.wrapDNNDealloc(base)


# (input shape, kernel, pads, strides): every window form the bf16 NHWC pooling kernels have --
# the compile-time 2x2 and 3x3 windows at strides 1 and 2, and the general loop (7x7, 1x1)
POOL16_CASES = [((2, 16, 12, 12), (2, 2), (0, 0), (2, 2)), ((2, 16, 13, 11), (3, 3), (1, 1), (2, 2)),
                ((1, 24, 9, 9), (3, 3), (1, 1), (1, 1)), ((2, 8, 7, 7), (7, 7), (0, 0), (1, 1)),
                ((1, 32, 10, 8), (2, 2), (0, 0), (1, 1)), ((2, 8, 6, 6), (1, 1), (0, 0), (1, 1)),
                ((1, 16, 9, 9), (5, 5), (2, 2), (2, 2))]


@pytest.mark.parametrize("mode", [rt.MATH_BF16, rt.MATH_F16])
@pytest.mark.parametrize("case", POOL16_CASES)
@pytest.mark.parametrize("avg", [False, True])
def test_pool_on_tensor_core_mode_activations(case, avg, mode):
    """Max and average pooling of a tensor that sits in the tensor-core mode's 16-bit NHWC
    format: the input is produced on the device by a 1x1 convolution, so the pool call takes
    the NHWC kernels (the fp32 NCHW ones are covered by test_pool).  Average pooling counts
    the padding in its divisor, like the reference's cuDNN descriptor
    (cudnn/CUDNNAveragePoolFunc.cpp:43-60)."""
    shape, k, p, s = case
    N, Cc, H, W = shape
    rt.set_math_mode(mode)
    r = rng(70 + H)
    x = r.uniform(-1, 1, shape).astype(np.float32)
    w = he(r, Cc, Cc, 1, 1)
    c0 = rt.counters()
    t = A.conv(A.up(x), A.up(w))
    y = A.pool(t, k, p, s, avg).numpy()
    c1 = rt.counters()
    assert c1["tc_launches"] - c0["tc_launches"] == 1      # the producer ran on the tensor cores
    tw = ref.conv2d(x, w)
    want = ref.pool2d(tw, k, p, s, avg=avg, count_include_pad=True)
    assert y.shape == want.shape
    assert max_rel_err(y, want) <= TOL[mode]
    # against the pool of exactly what the device pooled: only the output rounding is left
    t16 = t.numpy()
    exact = ref.pool2d(t16, k, p, s, avg=avg, count_include_pad=True)
    assert max_rel_err(y, exact) <= (STEP[mode] if avg else 0.0)


def test_reshape_is_a_copy():
    for mode in MODES:
        set_mode(mode)
        x = rng(13).normal(0, 1, (2, 8, 3, 5)).astype(np.float32)
        y = A.reshape(A.up(x), (2, 120)).numpy()
        assert np.array_equal(y, x.reshape(2, 120))
    # of a tensor-core mode tensor: NCHW order must come back (FC weights depend on it)
    rt.set_math_mode(rt.MATH_F16)
    r = rng(14)
    x = r.uniform(-1, 1, (2, 16, 4, 4)).astype(np.float32)
    w = he(r, 16, 16, 1, 1)
    t = A.conv(A.up(x), A.up(w))
    want = t.numpy().reshape(2, 256)
    assert np.array_equal(A.reshape(t, (2, 256)).numpy(), want)
    assert np.array_equal(A.flatten(t).numpy(), want)


def test_error_codes_for_bad_calls():
    """Compute entry points have no error channel in the reference ABI (the output pointer is
    returned whatever happened); here a bad call leaves a sticky code behind."""
    L = rt.lib()
    rt.set_math_mode(rt.MATH_BF16)
    x, w = A.Dev((1, 16, 4, 4)), A.Dev((8, 12, 1, 1))       # filter channels != input channels
    y = A.Dev((1, 8, 4, 4))
    L.DNNConvFunc(A.handle(), x.ptr, rt.dims(x.shape), w.ptr, rt.dims(w.shape), None, 0, 1, 1,
                  rt.dims((0, 0)), rt.dims((1, 1)), y.ptr)
    assert rt.last_error(clear=True) == 997
    a = A.Dev((2,) * 9)
    L.DNNTensorOpFunc(A.handle(), 0, a.ptr, rt.dims((2,) * 9), 9, a.ptr, rt.dims((2,) * 9), 9, a.ptr,
                      rt.dims((2,) * 9), 9, 1.0)
    assert rt.last_error(clear=True) == 996
    b = A.Dev((2, 3))
    L.DNNTensorOpFunc(A.handle(), 7, b.ptr, rt.dims((2, 3)), 2, b.ptr, rt.dims((2, 3)), 2, b.ptr,
                      rt.dims((2, 3)), 2, 1.0)               # op mode that does not exist
    assert rt.last_error(clear=True) == 996
    L.DNNReduceFunc(A.handle(), 2, b.ptr, rt.dims((2, 3)), b.ptr, rt.dims((2, 1)), 3)   # not the mean
    assert rt.last_error(clear=True) == 995


def test_reading_a_tensor_that_fusion_skipped_is_reported():
    """conv -> ReLU into a second tensor, twice: the second inference runs them as one kernel
    and never writes the convolution's own output.  A third inference that follows the same
    calls and then reads that output leaves the recorded sequence: the read is error 990."""
    import ctypes as C
    L = rt.lib()
    rt.set_math_mode(rt.MATH_BF16)
    r = rng(15)
    x = r.uniform(-1, 1, (1, 16, 6, 6)).astype(np.float32)
    w = he(r, 16, 16, 1, 1)
    n = 16 * 36 * 4

    def inference(read_conv_output):
        h, base = C.c_void_p(), C.c_void_p()
        L.cudnnCreate(C.byref(h))
        L.wrapDNNMemPoolInit(C.byref(base), 1 << 16)
        ptr = [C.c_void_p() for _ in range(4)]
        for i, nbytes in enumerate((n, w.nbytes, n, n)):
            L.wrapDNNMemOffset(C.byref(ptr[i]), base, i * 8192, nbytes)
        px, pw, pc, pr = ptr
        L.wrapDNNMemcpy(px, x.ctypes.data, n, 1, None)
        L.wrapDNNMemcpy(pw, w.ctypes.data, w.nbytes, 1, None)
        L.DNNConvFunc(h, px, rt.dims(x.shape), pw, rt.dims(w.shape), None, 0, 1, 1, rt.dims((0, 0)),
                      rt.dims((1, 1)), pc)
        L.DNNActiveFunc(h, pc, rt.dims(x.shape), 1, pr)
        out = np.empty(x.shape, np.float32)
        L.wrapDNNMemcpy(out.ctypes.data, pr, n, 2, None)
        conv_out = None
        if read_conv_output:
            conv_out = np.empty(x.shape, np.float32)
            L.wrapDNNMemcpy(conv_out.ctypes.data, pc, n, 2, None)
        L.wrapDNNDealloc(base)
        L.cudnnDestroy(h)
        return out, conv_out

    want = ref.conv2d(x, w, act=1)
    y0, _ = inference(False)
    chains = L.occamy_fused_chains()
    y1, _ = inference(False)
    assert L.occamy_fused_chains() == chains + 1
    assert max_rel_err(y0, want) <= 2e-2 and max_rel_err(y1, want) <= 2e-2
    assert rt.last_error(clear=True) == 0
    y2, _ = inference(True)
    assert max_rel_err(y2, want) <= 2e-2          # the fused result itself is fine
    assert rt.last_error(clear=True) == 990       # ... the skipped tensor is not there to read
    # that longer sequence is now a recorded program of its own: the convolution's output has a
    # second reader, so it is written again and the same calls succeed
    y3, c3 = inference(True)
    assert rt.last_error(clear=True) == 0
    assert max_rel_err(c3, ref.conv2d(x, w)) <= 2e-2 and max_rel_err(y3, want) <= 2e-2


def test_watchdog_turns_a_stuck_wait_into_an_error_code():
    """The kernels' waits are bounded: one that can never be satisfied ends after about two
    seconds with a code in the error word, and the context keeps working."""
    L = rt.lib()
    L.occamy_selftest_bounded_wait()
    rt.synchronize()
    assert rt.last_error(clear=True) == 1099
    # the stream and the context are still usable
    rt.set_math_mode(rt.MATH_BF16)
    r = rng(16)
    x = r.uniform(-1, 1, (1, 16, 5, 5)).astype(np.float32)
    w = he(r, 16, 16, 1, 1)
    y = A.conv(A.up(x), A.up(w)).numpy()
    assert max_rel_err(y, ref.conv2d(x, w)) <= 2e-2
    assert rt.last_error(clear=True) == 0


@pytest.mark.parametrize("bias_from", ["device_copy", "no_cache"])
def test_held_back_conv_with_a_bias_that_is_freed_early(bias_from):
    """conv -> in-place bias add -> (bias freed) -> ReLU, the order liveness-placed deallocs
    give.  From the second inference on the convolution is held back and takes the add along;
    when the bias has no resident copy (it was produced on the device, or the weight cache is
    off) the kernel reads the caller's bias tensor, so freeing that tensor has to run the
    held-back kernel first."""
    import ctypes as C
    L = rt.lib()
    rt.set_math_mode(rt.MATH_BF16)
    if bias_from == "no_cache":
        L.occamy_set_weight_cache(0)
    try:
        r = rng(17)
        x = r.uniform(-1, 1, (2, 32, 9, 9)).astype(np.float32)
        w = he(r, 32, 32, 3, 3)
        b = r.normal(0, 0.5, 32).astype(np.float32)
        want = ref.conv2d(x, w, b, (1, 1), (1, 1), act=1)

        def malloc(nbytes):
            p = C.c_void_p()
            L.wrapDNNMalloc(C.byref(p), nbytes)
            return p

        def inference():
            h = C.c_void_p()
            L.cudnnCreate(C.byref(h))
            px, pw, pb0, pb1 = malloc(x.nbytes), malloc(w.nbytes), malloc(b.nbytes), malloc(b.nbytes)
            pc, pr = malloc(x.nbytes), malloc(x.nbytes)
            L.wrapDNNMemcpy(px, x.ctypes.data, x.nbytes, 1, None)
            L.wrapDNNMemcpy(pw, w.ctypes.data, w.nbytes, 1, None)
            L.wrapDNNMemcpy(pb0, b.ctypes.data, b.nbytes, 1, None)
            bias = pb0
            if bias_from == "device_copy":
                L.wrapDNNMemcpy(pb1, pb0, b.nbytes, 3, None)
                bias = pb1
            L.DNNConvFunc(h, px, rt.dims(x.shape), pw, rt.dims(w.shape), None, 0, 1, 1,
                          rt.dims((1, 1)), rt.dims((1, 1)), pc)
            L.DNNTensorOpFunc(h, 0, pc, rt.dims(x.shape), 4, bias, rt.dims((1, 32, 1, 1)), 4, pc,
                              rt.dims(x.shape), 4, 1.0)
            L.wrapDNNDealloc(bias)                      # last use of the bias was the add
            # the freed bytes are handed out again and overwritten at once
            junk = malloc(b.nbytes)
            L.wrapDNNMemcpy(junk, (np.full(32, 1e6, np.float32)).ctypes.data, b.nbytes, 1, None)
            L.DNNActiveFunc(h, pc, rt.dims(x.shape), 1, pr)
            out = np.empty(x.shape, np.float32)
            L.wrapDNNMemcpy(out.ctypes.data, pr, out.nbytes, 2, None)
            for p in (px, pw, pc, pr, junk, pb1 if bias is pb0 else pb0):
                L.wrapDNNDealloc(p)
            L.cudnnDestroy(h)
            return out

        for i in range(3):
            y = inference()
            assert max_rel_err(y, want) <= 2e-2, i
            assert rt.last_error(clear=True) == 0
    finally:
        L.occamy_set_weight_cache(1)


def test_fp16_mode_is_finer_than_bf16_and_overflows_to_infinity():
    """The two 16-bit modes differ only in the element type: fp16 must be about eight times
    closer to the fp32 result on data of ordinary magnitude, and a value beyond fp16's range
    must come out as infinity (visible), not as a wrong finite number."""
    r = rng(18)
    x = r.uniform(-1, 1, (2, 64, 14, 14)).astype(np.float32)
    w = he(r, 64, 64, 3, 3)
    b = r.normal(0, 0.1, 64).astype(np.float32)
    want = ref.conv2d(x, w, b, (1, 1), (1, 1), act=5)
    errs = {}
    for mode in (rt.MATH_BF16, rt.MATH_F16):
        rt.set_math_mode(mode)
        y = A.conv(A.up(x), A.up(w), A.up(b), (1, 1), (1, 1), act_mode=5).numpy()
        errs[mode] = max_rel_err(y, want)
    assert errs[rt.MATH_F16] <= 2e-3 and errs[rt.MATH_F16] * 3 < errs[rt.MATH_BF16]
    rt.set_math_mode(rt.MATH_F16)
    big = A.conv(A.up(x * 1e4), A.up(w * 1e3), A.up(b), (1, 1), (1, 1), act_mode=5).numpy()
    assert np.isinf(big).any() and not np.isnan(big).any()
    # a tensor left in one 16-bit type is read correctly after the mode changes
    rt.set_math_mode(rt.MATH_BF16)
    t = A.conv(A.up(x), A.up(w), A.up(b), (1, 1), (1, 1), act_mode=1)
    rt.set_math_mode(rt.MATH_F16)
    u = A.active(t, 1).numpy()
    assert max_rel_err(u, np.maximum(want, 0)) <= 2e-2


# 1x1 layers large enough for the planner to choose 256-channel tiles, with at least 1024 input
# channels: they run as CTA pairs (two SMs per 256-pixel tile).  101 images of 14 x 14 give an
# odd number of 128-pixel tiles, so the last pair has only one real tile.
PAIR_CASES = [(100, 1024, 14, 14, 512, 1, 0), (101, 1024, 14, 14, 256, 1, 0), (200, 2048, 7, 7, 512, 1, 0),
              (33, 256, 14, 14, 256, 3, 1), (40, 512, 7, 7, 512, 3, 1)]


@pytest.mark.parametrize("mode", [rt.MATH_BF16, rt.MATH_F16])
@pytest.mark.parametrize("case", PAIR_CASES)
@pytest.mark.parametrize("act_mode", [1, 5])
def test_conv_on_cta_pairs(case, mode, act_mode):
    N, C, H, W, K, R, pad = case
    r = rng(hash(case) % 2**31)
    x = r.uniform(-1, 1, (N, C, H, W)).astype(np.float32)
    w = he(r, K, C, R, R)
    b = r.normal(0, 0.5, K).astype(np.float32)
    rt.set_math_mode(mode)
    y = A.conv(A.up(x), A.up(w), A.up(b), (pad, pad), (1, 1), 1, act_mode).numpy()
    want = ref.conv2d(x, w, b, (pad, pad), (1, 1), 1, act=act_mode)
    assert max_rel_err(y, want) <= TOL[mode]
    # every output pixel and channel was written by exactly the tile that owns it
    assert np.isfinite(y).all()
    err = np.abs(y - want).reshape(N, K, -1).max(axis=(1, 2)) / np.abs(want).max()
    assert err.max() <= TOL[mode]


# (N, C, H, W, stride): several strips per column, odd sizes, channel counts whose 16-byte pieces
# are not a power of two, images smaller than a strip, stride 2 with even and odd extents
DW_STRIP_CASES = [(2, 32, 33, 17, 1), (2, 96, 29, 29, 2), (1, 144, 56, 56, 1), (3, 8, 7, 7, 1),
                  (1, 24, 40, 12, 2), (2, 40, 112, 20, 1), (1, 960, 7, 7, 1), (2, 16, 3, 3, 1)]


@pytest.mark.parametrize("case", DW_STRIP_CASES)
def test_depthwise_fp16_register_strips(case):
    """fp16 mode runs 3x3 depthwise convolutions on packed fp16 pairs, a thread walking down a
    strip of rows: sums are kept in fp16, so the bound is tighter than the mode's 2e-2 but looser
    than one rounding (nine roundings to 11 bits plus the stored output's)."""
    N, C, H, W, st = case
    r = rng(hash(case) % 2**31)
    x = r.uniform(-1, 1, (N, C, H, W)).astype(np.float32)
    w = he(r, C, 1, 3, 3)
    rt.set_math_mode(rt.MATH_F16)
    c0 = rt.counters()
    y = A.conv(A.up(x), A.up(w), None, (1, 1), (st, st), C, None).numpy()
    assert rt.counters()["launches"] > c0["launches"]
    x16 = x.astype(np.float16).astype(np.float32)
    w16 = w.astype(np.float16).astype(np.float32)
    want = ref.conv2d(x16, w16, None, (1, 1), (st, st), C, act=5)
    assert y.shape == want.shape
    assert max_rel_err(y, want) <= 4e-3


# (N, C, H, W, K): layers with one channel tile and tiny weights (fetched once per CTA) and with
# 32-channel tiles (two CTAs per SM), large enough that every CTA walks through several tiles
FEW_CHANNEL_CASES = [(4, 32, 112, 112, 16), (2, 16, 112, 112, 96), (6, 144, 56, 56, 24),
                     (8, 96, 56, 56, 24), (16, 192, 28, 28, 32)]


@pytest.mark.parametrize("mode", [rt.MATH_BF16, rt.MATH_F16])
@pytest.mark.parametrize("case", FEW_CHANNEL_CASES)
@pytest.mark.parametrize("act_mode", [1, 3])
def test_conv_with_few_channels(case, mode, act_mode):
    N, C, H, W, K = case
    r = rng(hash(case) % 2**31)
    x = r.uniform(-1, 1, (N, C, H, W)).astype(np.float32)
    w = he(r, K, C, 1, 1)
    b = r.normal(0, 0.5, K).astype(np.float32)
    rt.set_math_mode(mode)
    y = A.conv(A.up(x), A.up(w), A.up(b), (0, 0), (1, 1), 1, act_mode).numpy()
    lo, hi = (0.0, 6.0) if act_mode == 3 else (0.0, 0.0)
    want = ref.conv2d(x, w, b, (0, 0), (1, 1), 1, act=act_mode, lo=lo, hi=hi)
    assert np.isfinite(y).all()
    # per image, so that a tile written to the wrong place or not at all cannot hide
    err = np.abs(y - want).reshape(N, -1).max(axis=1) / np.abs(want).max()
    assert err.max() <= TOL[mode]


def test_fp32_mode_runs_on_the_tensor_cores():
    """fp32 mode, dense 3x3 and 1x1 convolutions and the classifier GEMM: tensor-core launches
    are counted, no CUDA-core convolution / GEMM launch is, and the result is within the fp32
    bound with room to spare (the split operands carry all 24 mantissa bits)."""
    rt.set_math_mode(rt.MATH_FP32)
    r = rng(19)
    x = r.uniform(-1, 1, (4, 96, 28, 28)).astype(np.float32)
    w3, w1 = he(r, 128, 96, 3, 3), he(r, 64, 128, 1, 1)
    b3, b1 = r.normal(0, 0.3, 128).astype(np.float32), r.normal(0, 0.3, 64).astype(np.float32)
    c0 = rt.counters()
    t = A.conv(A.up(x), A.up(w3), A.up(b3), (1, 1), (2, 2), act_mode=1)
    y = A.conv(t, A.up(w1), A.up(b1), act_mode=5).numpy()
    a = r.normal(0, 1, (64, 500)).astype(np.float32)
    bm = (r.normal(0, 1, (200, 500)) / 22).astype(np.float32)
    m = A.matmul2d(A.up(a), A.up(bm), 1.0, 1.0, 0, 1).numpy()
    c1 = rt.counters()
    assert c1["tc_launches"] - c0["tc_launches"] == 3
    assert c1["simt_launches"] == c0["simt_launches"]
    want = ref.conv2d(ref.conv2d(x, w3, b3, (1, 1), (2, 2), act=1), w1, b1, act=5)
    assert max_rel_err(y, want) <= 2e-5
    assert max_rel_err(m, ref.matmul2d(a, bm, None, 1.0, 0.0, 0, 1)) <= 2e-5


def test_constant_changed_in_place_is_noticed():
    """A filter uploaded from host memory is recognised at its next upload (same address, same
    size) and its packed copy reused.  The fingerprint behind that samples the whole buffer, so
    a constant whose interior changed -- its first and last 512 bytes untouched -- is packed
    again instead of being served from the stale copy."""
    import ctypes as C
    L = rt.lib()
    rt.set_math_mode(rt.MATH_BF16)
    r = rng(20)
    x = r.uniform(-1, 1, (1, 64, 12, 12)).astype(np.float32)
    w = he(r, 64, 64, 3, 3)                      # 147 KB: head and tail are 0.7 % of it
    xd = A.up(x)

    def run():
        h = C.c_void_p()
        L.cudnnCreate(C.byref(h))
        wd, y = C.c_void_p(), A.Dev((1, 64, 12, 12))
        L.wrapDNNMalloc(C.byref(wd), w.nbytes)
        L.wrapDNNMemcpy(wd, w.ctypes.data, w.nbytes, 1, None)      # same host address every time
        L.DNNConvFunc(h, xd.ptr, rt.dims(x.shape), wd, rt.dims(w.shape), None, 0, 1, 1,
                      rt.dims((1, 1)), rt.dims((1, 1)), y.ptr)
        out = y.numpy()
        L.wrapDNNDealloc(wd)
        L.cudnnDestroy(h)
        return out

    y0 = run()
    c0 = rt.counters()
    y1 = run()
    assert np.array_equal(y0, y1)
    assert rt.counters()["h2d_skipped_bytes"] - c0["h2d_skipped_bytes"] == w.nbytes   # reused
    flat = w.reshape(-1)
    flat[128:-128] *= -2.0                        # interior only
    y2 = run()
    want = ref.conv2d(x, w, None, (1, 1), (1, 1))
    assert max_rel_err(y2, want) <= 2e-2


GUARD_CASES = [("conv", (1, 32, 13, 11, 24, 3, 1, 1)), ("conv", (3, 512, 7, 7, 512, 3, 1, 1)),
               ("conv", (2, 24, 14, 14, 144, 1, 0, 1)), ("conv", (2, 3, 64, 64, 64, 7, 3, 2)),
               ("conv", (2, 256, 28, 28, 128, 1, 0, 2)), ("depthwise", (2, 96, 15, 15, 96, 3, 1, 2)),
               ("pool", (2, 16, 13, 11)), ("add", (2, 40, 9, 7))]


@pytest.mark.parametrize("mode", [rt.MATH_FP32, rt.MATH_BF16, rt.MATH_F16])
@pytest.mark.parametrize("case", GUARD_CASES)
def test_kernels_write_nothing_outside_their_output(case, mode):
    """Stands in for a memory checker: the output tensor sits inside a larger allocation whose
    bytes before and after it hold a pattern; after the call the pattern must be intact.
    Ragged shapes on purpose (tiles that overhang the tensor, channel counts below a tile)."""
    import ctypes as C
    L = rt.lib()
    kind, shp = case
    set_mode(mode)
    r = rng(21)
    GUARD = 4096                                   # bytes on either side
    pattern = np.full(GUARD // 4, -7.25e33, np.float32)

    def guarded(nbytes):
        base = C.c_void_p()
        L.wrapDNNMalloc(C.byref(base), GUARD + nbytes + GUARD)
        L.wrapDNNMemcpy(base, pattern.ctypes.data, GUARD, 1, None)
        L.wrapDNNMemcpy(base.value + GUARD + nbytes, pattern.ctypes.data, GUARD, 1, None)
        return base, C.c_void_p(base.value + GUARD)

    def guards_intact(base, nbytes):
        lo, hi = np.empty_like(pattern), np.empty_like(pattern)
        L.wrapDNNMemcpy(lo.ctypes.data, base, GUARD, 2, None)
        L.wrapDNNMemcpy(hi.ctypes.data, base.value + GUARD + nbytes, GUARD, 2, None)
        return np.array_equal(lo, pattern) and np.array_equal(hi, pattern)

    if kind in ("conv", "depthwise"):
        N, Cc, H, W, K, R, pad, stride = shp
        groups = Cc if kind == "depthwise" else 1
        x = r.uniform(-1, 1, (N, Cc, H, W)).astype(np.float32)
        w = he(r, K, Cc // groups, R, R)
        P = (H + 2 * pad - R) // stride + 1
        Q = (W + 2 * pad - R) // stride + 1
        nbytes = N * K * P * Q * 4
        base, y = guarded(nbytes)
        xd, wd = A.up(x), A.up(w)
        L.DNNConvFunc(A.handle(), xd.ptr, rt.dims(x.shape), wd.ptr, rt.dims(w.shape), None, 0, 1,
                      groups, rt.dims((pad, pad)), rt.dims((stride, stride)), y)
        want = ref.conv2d(x, w, None, (pad, pad), (stride, stride), groups)
    elif kind == "pool":
        x = r.uniform(-1, 1, shp).astype(np.float32)
        N, Cc, H, W = shp
        w1 = he(r, Cc, Cc, 1, 1)
        t = A.conv(A.up(x), A.up(w1))               # a 16-bit tensor in the 16-bit modes
        P, Q = (H + 2 - 3) // 2 + 1, (W + 2 - 3) // 2 + 1
        nbytes = N * Cc * P * Q * 4
        base, y = guarded(nbytes)
        L.DNNMaxPoolFunc(A.handle(), t.ptr, rt.dims(shp), y, rt.dims((N, Cc, P, Q)), rt.dims((3, 3)),
                         rt.dims((1, 1, 1, 1)), rt.dims((2, 2)))
        want = ref.pool2d(ref.conv2d(x, w1), (3, 3), (1, 1), (2, 2))
    else:
        x = r.uniform(-1, 1, shp).astype(np.float32)
        N, Cc, H, W = shp
        w1 = he(r, Cc, Cc, 1, 1)
        t = A.conv(A.up(x), A.up(w1))
        nbytes = x.nbytes
        base, y = guarded(nbytes)
        L.DNNTensorOpFunc(A.handle(), 0, t.ptr, rt.dims(shp), 4, t.ptr, rt.dims(shp), 4, y,
                          rt.dims(shp), 4, 1.0)
        want = 2 * ref.conv2d(x, w1)
    got = np.empty(want.shape, np.float32)
    L.wrapDNNMemcpy(got.ctypes.data, y, got.nbytes, 2, None)
    assert max_rel_err(got, want) <= TOL[mode]
    assert guards_intact(base, nbytes)
    L.wrapDNNDealloc(base)
