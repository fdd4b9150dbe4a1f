"""Whole-graph parity on a B200: the replayed runtime-call program of each benchmark graph
against the CPU oracle evaluating the same graph on the same seeded tensors.

fp32 mode: max relative error <= 1e-4 per output tensor.
16-bit tensor-core modes: <= 2e-2 relative on the logits and identical top-1 indices -- bf16 for
ResNet-50 and VGG-16, fp16 for MobileNetV2.  (Why not bf16 there: tests/test_mode_choice.py
shows on the CPU that rounding nothing but the weights of this random-weight MobileNetV2 to
bf16 already moves its logits by more than 2e-2.)
"""
import numpy as np
import pytest

from helpers import max_rel_err, run_graph_oracle, top1_agrees
from occamy_b200 import graphs, replay
from occamy_b200 import runtime as rt

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _check_runtime_errors(native_libs):
    rt.last_error(clear=True)
    yield
    rt.synchronize()
    assert rt.last_error(clear=True) == 0


def run_both(g, x, mode, fuse, pool_opt=True, dealloc_opt=True, repeats=1):
    rt.set_math_mode(mode)
    p = g.to_program()
    p.lower(fuse=fuse, dealloc_opt=dealloc_opt, pool_opt=pool_opt)
    b = replay.Binding()
    outs = None
    for _ in range(repeats):
        outs = p.run(b, x)
    return outs, p


def check_logits(y, want, mode, bf16_tol=2e-2):
    if mode == rt.MATH_FP32:
        assert max_rel_err(y, want) <= 1e-4
    else:
        assert max_rel_err(y, want) <= bf16_tol
    ok, ties = top1_agrees(y, want)
    assert ok and ties == 0


@pytest.mark.parametrize("mode", [rt.MATH_FP32, rt.MATH_BF16])
@pytest.mark.parametrize("fuse", [replay.FUSE_NONE, replay.FUSE_REFERENCE])
def test_single_conv_config(mode, fuse):
    g = graphs.single_conv(seed=0)
    x = graphs.make_input(g, 0, "uniform")
    (y,), _ = run_both(g, x, mode, fuse)
    (want,) = run_graph_oracle(g, x)
    assert max_rel_err(y, want) <= (1e-4 if mode == rt.MATH_FP32 else 2e-2)


@pytest.mark.parametrize("mode", [rt.MATH_FP32, rt.MATH_BF16])
@pytest.mark.parametrize("variant", ["v1", "v1.5"])
def test_resnet50_batch2(mode, variant):
    g = graphs.resnet50(batch=2, seed=0, variant=variant, softmax=False)
    x = graphs.make_input(g, 0)
    # run twice: the second inference takes the resident-weight path
    (y,), p = run_both(g, x, mode, replay.FUSE_REFERENCE, repeats=2)
    (want,) = run_graph_oracle(g, x)
    check_logits(y, want, mode)


@pytest.mark.parametrize("mode", [rt.MATH_FP32, rt.MATH_BF16])
def test_resnet50_unfused_no_pool_softmax(mode):
    """What the reference's own test scripts compile: no fusion; here also without the
    pool, so every tensor is its own wrapDNNMalloc / wrapDNNDealloc."""
    g = graphs.resnet50(batch=1, seed=1, variant="v1", softmax=True, image=64)
    x = graphs.make_input(g, 1)
    (y,), _ = run_both(g, x, mode, replay.FUSE_NONE, pool_opt=False)
    (want,) = run_graph_oracle(g, x)
    assert max_rel_err(y, want) <= (1e-4 if mode == rt.MATH_FP32 else 2e-2)
    assert np.array_equal(y.argmax(1), want.argmax(1))
    np.testing.assert_allclose(y.sum(1), 1.0, rtol=1e-5)


@pytest.mark.parametrize("mode", [rt.MATH_FP32, rt.MATH_F16])
@pytest.mark.parametrize("fuse", [replay.FUSE_NONE, replay.FUSE_WITH_CLIP])
def test_mobilenet_v2(mode, fuse):
    g = graphs.mobilenet_v2(batch=2, seed=0, image=96)
    x = graphs.make_input(g, 0)
    (y,), _ = run_both(g, x, mode, fuse, repeats=2)
    (want,) = run_graph_oracle(g, x)
    check_logits(y, want, mode)


def test_mobilenet_v2_bf16_runs_and_keeps_top1():
    """bf16 mode on this network is outside the 2e-2 contract (8 mantissa bits are not enough,
    whatever the kernels do) but it must still run and rank the classes the same way."""
    g = graphs.mobilenet_v2(batch=2, seed=0, image=96)
    x = graphs.make_input(g, 0)
    (y,), _ = run_both(g, x, rt.MATH_BF16, replay.FUSE_WITH_CLIP, repeats=2)
    (want,) = run_graph_oracle(g, x)
    assert max_rel_err(y, want) <= 8e-2
    assert top1_agrees(y, want)[0]


@pytest.mark.parametrize("mode", [rt.MATH_FP32, rt.MATH_BF16])
def test_vgg16_small_image(mode):
    g = graphs.vgg16(batch=2, seed=0, image=64, num_classes=100)
    x = graphs.make_input(g, 0)
    (y,), p = run_both(g, x, mode, replay.FUSE_REFERENCE)
    (want,) = run_graph_oracle(g, x)
    check_logits(y, want, mode)
    assert rt.counters()["pool_hwm_bytes"] >= p.pool_bytes


def test_resident_weights_skip_uploads():
    """After the first inference the constants' packed forms are resident: the second
    inference uploads (almost) nothing but the input batch and gives the same bits."""
    rt.set_math_mode(rt.MATH_BF16)
    g = graphs.resnet50(batch=1, seed=2, softmax=False, image=64)
    x = graphs.make_input(g, 2)
    p = g.to_program()
    p.lower(fuse=replay.FUSE_REFERENCE)
    b = replay.Binding()
    p.run(b, x)                       # first inference: packs weights, records the calls
    (y1,) = p.run(b, x)
    c1 = rt.counters()
    (y2,) = p.run(b, x)
    c2 = rt.counters()
    assert np.array_equal(y1, y2)
    uploaded = c2["h2d_bytes"] - c1["h2d_bytes"]
    skipped = c2["h2d_skipped_bytes"] - c1["h2d_skipped_bytes"]
    assert skipped > 90e6 and uploaded < x.nbytes + 1e6
    assert c2["tc_launches"] - c1["tc_launches"] == 54   # 53 convolutions + the classifier


def test_deterministic_replay():
    rt.set_math_mode(rt.MATH_BF16)
    g = graphs.resnet50(batch=2, seed=3, softmax=False, image=96)
    x = graphs.make_input(g, 3)
    p = g.to_program()
    p.lower(fuse=replay.FUSE_REFERENCE)
    b = replay.Binding()
    outs = [p.run(b, x)[0] for _ in range(4)]
    # the first inference runs call by call, later ones fold add / ReLU calls into the
    # convolutions (fewer bf16 roundings): identical from the second on
    assert np.array_equal(outs[1], outs[2]) and np.array_equal(outs[2], outs[3])
    assert max_rel_err(outs[0], outs[1]) <= 1e-2


@pytest.mark.parametrize("case", [("resnet50", replay.FUSE_REFERENCE, 17),
                                  ("resnet50", replay.FUSE_NONE, 53),
                                  ("mobilenet_v2", replay.FUSE_NONE, 52),
                                  ("mobilenet_v2", replay.FUSE_REFERENCE, 45)])
def test_cross_call_fusion(case):
    """Element-wise calls that follow a convolution are folded into its epilogue once the
    call sequence has been seen: conv3 + residual add + ReLU of every ResNet block with the
    reference's fusion on (plus the stem convolution with its max pool); conv + bias add +
    ReLU/Clip (+ residual) without it."""
    name, fuse, chains = case
    rt.set_math_mode(rt.MATH_BF16 if name == "resnet50" else rt.MATH_F16)
    g = getattr(graphs, name)(batch=2, seed=4, image=64)
    x = graphs.make_input(g, 4)
    p = g.to_program()
    p.lower(fuse=fuse)
    b = replay.Binding()
    (want,) = run_graph_oracle(g, x)
    (y0,) = p.run(b, x)
    n0 = rt.lib().occamy_fused_chains()
    launches0 = rt.counters()["launches"]
    (y1,) = p.run(b, x)
    n1 = rt.lib().occamy_fused_chains()
    launches1 = rt.counters()["launches"]
    (y2,) = p.run(b, x)
    assert n1 - n0 == chains
    assert np.array_equal(y1, y2)
    assert max_rel_err(y0, want) <= 2e-2 and max_rel_err(y1, want) <= 2e-2
    assert top1_agrees(y1, want) == (True, 0)
    # the fused replay issues fewer kernels than the call-by-call one
    p2 = g.to_program()
    p2.lower(fuse=fuse)
    rt.lib().occamy_set_cross_call_fusion(0)
    try:
        before = rt.counters()["launches"]
        (y3,) = p2.run(b, x)
        eager_launches = rt.counters()["launches"] - before
    finally:
        rt.lib().occamy_set_cross_call_fusion(1)
    assert launches1 - launches0 < eager_launches
    assert np.array_equal(y3, y0)


def test_new_call_sequence_after_a_recorded_one():
    """A different program after a recorded one simply runs call by call first."""
    rt.set_math_mode(rt.MATH_BF16)
    b = replay.Binding()
    ga = graphs.resnet50(batch=1, seed=5, image=64, softmax=False)
    gb = graphs.resnet50(batch=2, seed=5, image=64, softmax=False)
    xa, xb = graphs.make_input(ga, 5), graphs.make_input(gb, 5)
    pa, pb = ga.to_program(), gb.to_program()
    pa.lower()
    pb.lower()
    (a1,) = pa.run(b, xa)
    (a2,) = pa.run(b, xa)
    (b1,) = pb.run(b, xb)
    (a3,) = pa.run(b, xa)
    (b2,) = pb.run(b, xb)
    assert np.array_equal(a2, a3)
    (wa,) = run_graph_oracle(ga, xa)
    (wb,) = run_graph_oracle(gb, xb)
    for y, w in ((a1, wa), (a3, wa), (b1, wb), (b2, wb)):
        assert max_rel_err(y, w) <= 2e-2


def _stem_graph(N, H, W, R, pad, act, seed):
    g = graphs.Graph((N, 3, H, W), seed)
    g.name = "stem"
    w, b = g.he_conv(64, 3, R, R)
    y = g.conv(0, w, b, pads=(pad, pad), strides=(2, 2))
    if act == "relu":
        y = g.relu(y)
    elif act == "clip":
        y = g.clip(y, -0.25, 0.75)
    y = g.maxpool(y, (3, 3), (1, 1), (2, 2))
    g.mark_output(y)
    return g


@pytest.mark.parametrize("shape", [(2, 64, 64, 7, 3, "relu"), (3, 224, 224, 7, 3, "relu"),
                                   (1, 70, 54, 7, 3, "clip"), (2, 33, 47, 5, 2, "none"),
                                   (5, 96, 200, 3, 1, "relu"), (1, 17, 250, 7, 3, "relu")])
@pytest.mark.parametrize("fuse", [replay.FUSE_REFERENCE, replay.FUSE_NONE])
def test_stem_conv_with_max_pool(shape, fuse):
    """A 64-channel RGB stem and the 3x3 / stride 2 max pool behind it run as one kernel from
    the second inference on; the result must match the call-by-call run bit for bit (same
    bf16 rounding of the convolution output before the pool) and the oracle within the bf16
    tolerance.  Odd sizes exercise the image edges of both the convolution and the pool."""
    N, H, W, R, pad, act = shape
    rt.set_math_mode(rt.MATH_BF16)
    g = _stem_graph(N, H, W, R, pad, act, seed=7)
    x = graphs.make_input(g, 5)
    p = g.to_program()
    p.lower(fuse=fuse)
    b = replay.Binding()
    (want,) = run_graph_oracle(g, x)
    (y0,) = p.run(b, x)
    n0 = rt.lib().occamy_fused_chains()
    (y1,) = p.run(b, x)
    assert rt.lib().occamy_fused_chains() - n0 == 1
    assert rt.last_error() == 0
    assert max_rel_err(y0, want) <= 2e-2 and max_rel_err(y1, want) <= 2e-2
    # conv + ReLU fused by the reference lowering round the same way in both runs
    if fuse == replay.FUSE_REFERENCE and act != "clip":
        assert np.array_equal(y0, y1)


@pytest.mark.parametrize("name", ["resnet50", "mobilenet_v2"])
def test_offline_pool_plan_runs_the_same(name):
    """The runtime takes whatever offsets the caller planned: with the greedy-by-size plan
    (smaller pool, different aliasing between tensors) the result is the same bits as with
    the reference's first-fit plan, call by call and with cross-call fusion."""
    rt.set_math_mode(rt.MATH_BF16 if name == "resnet50" else rt.MATH_F16)
    g = getattr(graphs, name)(batch=2, seed=5, image=64)
    x = graphs.make_input(g, 6)
    b = replay.Binding()
    outs = {}
    for mode in (replay.POOL_FIRST_FIT, replay.POOL_BY_SIZE):
        p = g.to_program()
        p.lower(fuse=replay.FUSE_REFERENCE, pool_opt=mode)
        outs[mode] = [p.run(b, x)[0] for _ in range(3)]
        assert rt.last_error() == 0
        assert np.array_equal(outs[mode][1], outs[mode][2])
    assert np.array_equal(outs[replay.POOL_FIRST_FIT][0], outs[replay.POOL_BY_SIZE][0])
    assert np.array_equal(outs[replay.POOL_FIRST_FIT][2], outs[replay.POOL_BY_SIZE][2])
