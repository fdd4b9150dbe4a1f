"""Whole-graph parity on a B200: the replayed runtime-call program of each benchmark graph
against the CPU oracle evaluating the same graph on the same seeded tensors.

fp32 mode: max relative error <= 1e-4 per output tensor.
bf16 tensor-core mode: <= 2e-2 relative on the logits and identical top-1 indices.
"""
import numpy as np
import pytest

from helpers import max_rel_err, run_graph_oracle
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
    assert np.array_equal(y.argmax(1), want.argmax(1))


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


@pytest.mark.parametrize("mode", [rt.MATH_FP32, rt.MATH_BF16])
@pytest.mark.parametrize("fuse", [replay.FUSE_NONE, replay.FUSE_WITH_CLIP])
def test_mobilenet_v2(mode, fuse):
    g = graphs.mobilenet_v2(batch=2, seed=0, image=96)
    x = graphs.make_input(g, 0)
    (y,), _ = run_both(g, x, mode, fuse)
    (want,) = run_graph_oracle(g, x)
    # bf16 activation storage alone (emulated on the CPU: every tensor rounded to bf16, fp32
    # arithmetic) puts this 53-layer random-weight network 4.8e-2 from the fp32 result, so the
    # 2e-2 bound that holds for ResNet-50 and VGG-16 cannot hold here; top-1 must still agree.
    check_logits(y, want, mode, bf16_tol=8e-2)


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
    outs = [p.run(b, x)[0] for _ in range(3)]
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[1], outs[2])
