"""The benchmark configurations at their stated shapes on a B200: ResNet-50 batch 256,
MobileNetV2 batch 128 and VGG-16 batch 64 (1000 classes, 224 x 224 images), the whole batch
through the replayed runtime-call program, compared with the CPU oracle on a few images of
that batch (images are independent: no operator of these graphs mixes samples, so the oracle
evaluates the same graph built for the sampled images only, same seeded weights).

fp32 mode: max relative error <= 1e-4 on the logits.
16-bit tensor-core mode: <= 2e-2 on the logits and identical top-1 indices.
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


def full_batch_vs_sampled_oracle(builder, batch, sample, mode, tol, repeats=2, **kw):
    rt.set_math_mode(mode)
    g = builder(batch=batch, seed=0, **kw)
    x = graphs.make_input(g, 0)
    p = g.to_program()
    p.lower(fuse=replay.FUSE_REFERENCE)
    b = replay.Binding()
    y = None
    for _ in range(repeats):          # the second inference runs the recorded, fused sequence
        (y,) = p.run(b, x)
    assert y.shape[0] == batch and np.isfinite(y).all()
    gs = builder(batch=len(sample), seed=0, **kw)
    (want,) = run_graph_oracle(gs, x[list(sample)])
    got = y[list(sample)]
    err = max_rel_err(got, want)
    assert err <= tol, err
    ok, ties = top1_agrees(got, want)
    assert ok and ties <= len(sample) // 3, (got.argmax(1), want.argmax(1), ties)
    return p, y


@pytest.mark.parametrize("mode", [rt.MATH_FP32, rt.MATH_BF16])
def test_resnet50_batch256(mode):
    c0 = rt.counters()
    p, y = full_batch_vs_sampled_oracle(graphs.resnet50, 256, (0, 85, 170, 255), mode,
                                        1e-4 if mode == rt.MATH_FP32 else 2e-2, softmax=False)
    c1 = rt.counters()
    if mode == rt.MATH_BF16:
        assert c1["tc_launches"] - c0["tc_launches"] == 2 * 54
    assert c1["pool_hwm_bytes"] >= p.pool_bytes


@pytest.mark.parametrize("mode", [rt.MATH_FP32, rt.MATH_F16])
def test_mobilenet_v2_batch128(mode):
    full_batch_vs_sampled_oracle(graphs.mobilenet_v2, 128, (0, 42, 127), mode,
                                 1e-4 if mode == rt.MATH_FP32 else 2e-2)


@pytest.mark.parametrize("mode", [rt.MATH_FP32, rt.MATH_BF16])
def test_vgg16_batch64(mode):
    """25088 -> 4096 first FC layer, the 822 MB [64,64,224,224] activation and the planner's
    peak: the pool the replayed program asks for is the one the runtime serves."""
    p, y = full_batch_vs_sampled_oracle(graphs.vgg16, 64, (0, 21, 42, 63), mode,
                                        1e-4 if mode == rt.MATH_FP32 else 2e-2, repeats=1)
    assert y.shape == (64, 1000)
    assert rt.counters()["pool_hwm_bytes"] >= p.pool_bytes >= 64 * 64 * 224 * 224 * 4
