"""Pins the CPU oracle: against golden vectors computed independently (torch float64,
tests/golden/make_golden.py) and against torch.nn.functional on edge cases.  The reference
repository itself holds no golden vectors for this path."""
import os

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from helpers import max_rel_err, run_graph_oracle
from occamy_b200 import graphs
from oracle import ref

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "ops_golden.npz"))


def test_golden_single_conv_config():
    g = graphs.single_conv(seed=0)
    x = graphs.make_input(g, 0, "uniform")
    (y,) = run_graph_oracle(g, x)
    assert max_rel_err(y[:, ::4, ::7, ::7], GOLD["c1_sample"]) <= 2e-6
    np.testing.assert_allclose([y.sum(dtype=np.float64), np.abs(y).sum(dtype=np.float64)],
                               GOLD["c1_sum"], rtol=1e-5)


@pytest.mark.parametrize("variant", ["v1", "v1.5"])
def test_golden_resnet50_logits(variant):
    g = graphs.resnet50(batch=2, seed=0, variant=variant, softmax=False)
    (y,) = run_graph_oracle(g, graphs.make_input(g, 0))
    want = GOLD[f"resnet50_{variant}_b2_logits"]
    assert max_rel_err(y, want) <= 1e-4
    assert np.array_equal(y.argmax(1), want.argmax(1))


def test_golden_mobilenet_and_vgg_logits():
    g = graphs.mobilenet_v2(batch=2, seed=0, image=96)
    (y,) = run_graph_oracle(g, graphs.make_input(g, 0))
    assert max_rel_err(y, GOLD["mobilenet_v2_b2_i96_logits"]) <= 1e-4
    g = graphs.vgg16(batch=2, seed=0, image=64, num_classes=100)
    (y,) = run_graph_oracle(g, graphs.make_input(g, 0))
    assert max_rel_err(y, GOLD["vgg16_b2_i64_logits"]) <= 1e-4


def test_golden_single_ops():
    x, w, b = GOLD["op_x"], GOLD["op_w"], GOLD["op_b"]
    assert max_rel_err(ref.conv2d(x, w, b, (1, 1), (2, 2), 2), GOLD["op_conv_g2_s2_p1"]) <= 1e-6
    assert max_rel_err(ref.conv2d(x, w, b, (1, 1), (2, 2), 2, f64=True),
                       GOLD["op_conv_g2_s2_p1"]) <= 1e-7
    assert max_rel_err(ref.pool2d(x, (3, 3), (1, 1), (2, 2)), GOLD["op_maxpool_3s2p1"]) == 0
    assert max_rel_err(ref.pool2d(x, (3, 3), (1, 1), (2, 2), avg=True),
                       GOLD["op_avgpool_3s2p1_incl"]) <= 1e-6
    assert max_rel_err(ref.softmax(x, 1), GOLD["op_softmax_axis1"]) <= 1e-6


@pytest.mark.parametrize("N,C,H,W,K,R,pad,stride,groups", [
    (1, 1, 1, 1, 1, 1, 0, 1, 1), (2, 4, 5, 7, 6, 3, 1, 1, 2), (1, 3, 11, 11, 5, 7, 3, 2, 1),
    (3, 8, 6, 6, 8, 3, 1, 2, 8), (1, 2, 4, 4, 2, 4, 0, 1, 1), (2, 6, 9, 9, 4, 5, 2, 3, 1)])
def test_conv_against_torch(N, C, H, W, K, R, pad, stride, groups):
    r = np.random.Generator(np.random.PCG64(N * 100 + C))
    x = r.normal(0, 1, (N, C, H, W)).astype(np.float32)
    w = r.normal(0, 1, (K, C // groups, R, R)).astype(np.float32)
    b = r.normal(0, 1, K).astype(np.float32)
    want = F.conv2d(torch.tensor(x).double(), torch.tensor(w).double(), torch.tensor(b).double(),
                    stride, pad, 1, groups).numpy()
    for act, fn in ((5, lambda v: v), (1, lambda v: np.maximum(v, 0)),
                    (3, lambda v: np.clip(v, 0, 6))):
        y = ref.conv2d(x, w, b, (pad, pad), (stride, stride), groups, act=act, lo=0.0, hi=6.0)
        assert max_rel_err(y, fn(want)) <= 1e-5


def test_avgpool_count_exclude_pad_matches_onnx_default():
    x = np.random.default_rng(0).normal(0, 1, (1, 2, 5, 5)).astype(np.float32)
    y = ref.pool2d(x, (3, 3), (1, 1), (1, 1), avg=True, count_include_pad=False)
    want = F.avg_pool2d(torch.tensor(x), 3, 1, 1, count_include_pad=False).numpy()
    assert max_rel_err(y, want) <= 1e-6


def test_tensor_op_and_reduce_and_gemm():
    r = np.random.default_rng(1)
    a = r.normal(0, 1, (2, 3, 4, 5)).astype(np.float32)
    b = r.normal(0, 1, (1, 3, 1, 1)).astype(np.float32)
    np.testing.assert_allclose(ref.tensor_op(0, a, b, 2.0), a + 2.0 * b, rtol=1e-6)
    np.testing.assert_allclose(ref.tensor_op(1, a, b), a * b, rtol=1e-6)
    np.testing.assert_allclose(ref.reduce_mean(a, (2, 1, 4, 1)), a.mean((1, 3), keepdims=True),
                               rtol=1e-5, atol=1e-6)
    A, B = r.normal(0, 1, (4, 6)).astype(np.float32), r.normal(0, 1, (6, 5)).astype(np.float32)
    C0 = r.normal(0, 1, (4, 5)).astype(np.float32)
    np.testing.assert_allclose(ref.matmul2d(A, B, C0, 0.5, 2.0), 0.5 * A @ B + 2 * C0, rtol=1e-5,
                               atol=1e-6)
    np.testing.assert_allclose(ref.matmul2d(A.T.copy(), B.T.copy(), transA=1, transB=1), A @ B,
                               rtol=1e-5, atol=1e-6)


def test_relu_propagates_nan_and_softmax_is_shift_invariant():
    x = np.array([np.nan, -1.0, 2.0], np.float32)
    y = ref.activation(x, 1)
    assert np.isnan(y[0]) and y[1] == 0 and y[2] == 2
    z = np.random.default_rng(2).normal(0, 1, (3, 9)).astype(np.float32)
    np.testing.assert_allclose(ref.softmax(z, 1), ref.softmax(z + 50.0, 1), rtol=2e-5)
