"""Pins the CPU oracle against the reference's own runtime: the cuDNN / cuBLASLt wrappers of
corelab-src/occamy, compiled unchanged into oracle/_ref/ by oracle/build.py, replayed with
the same call programs.  Skipped when that library was not built.

Each replay runs in a child process whose environment carries NVIDIA_TF32_OVERRIDE=0, the
library switch that keeps cuDNN's and cuBLAS's fp32 paths off the TF32 tensor cores, so the
reference computes in true fp32 (cudnn/CUDNNConvFunc.cpp:70, cublas/CUBLASMatmul2dFunc.cu:73)
and the oracle must agree with it to the fp32 bound, 1e-4 per tensor, not to a TF32 one.
"""
import os
import subprocess
import sys

import numpy as np
import pytest

from helpers import max_rel_err, run_graph_oracle
from occamy_b200 import graphs, replay
from oracle import build as obuild

import ref_wrapper_run

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-4


def reference_outputs(tmp_path, name, batch=1, image=0, fuse=replay.FUSE_NONE, workspace=1 << 20):
    if not os.path.exists(obuild.REF_SO):
        pytest.skip("reference wrappers not built (oracle/_ref)")
    out = os.path.join(str(tmp_path), f"{name}.npz")
    env = dict(os.environ, NVIDIA_TF32_OVERRIDE="0")
    r = subprocess.run([sys.executable, ref_wrapper_run.__file__, name, str(batch), str(image),
                        str(int(fuse)), str(int(workspace)), out], env=env, capture_output=True,
                       text=True, timeout=600)
    if r.returncode != 0 and ("cannot bind" in r.stderr or "cannot open shared object" in r.stderr):
        pytest.skip(f"reference wrappers do not load here: {r.stderr[-300:]}")
    assert r.returncode == 0, r.stderr[-2000:]
    with np.load(out) as z:
        return [z[k] for k in z.files]


def oracle_outputs(name, batch, image, reference_gpu_gemm=True):
    """The oracle on the same graph.  One quirk of the reference's GPU path is modelled here,
    not in the oracle: a Gemm's C operand never reaches the output there.  The lowering adds
    it with a rank-2 DNNTensorOpFunc call (ONNXToDNN/Ops/cublas/Gemm.cpp:67-73), the wrapper
    hands rank-2 shapes to cudnnSetTensorNdDescriptor, which refuses fewer than three
    dimensions, and the failed cudnnOpTensor's status is dropped
    (cudnn/CUDNNTensorOpFunc.cpp:86-124).  The reference's CPU lowering, which is what this
    runtime has to match, does add C; so does the oracle everywhere else."""
    g, dist = ref_wrapper_run.build_graph(name, batch, image)
    if reference_gpu_gemm:
        for n in g.nodes:
            if n.op == "gemm":
                n.ins = (n.ins[0], n.ins[1], -1)
    x = graphs.make_input(g, 0, dist)
    return run_graph_oracle(g, x)


@pytest.mark.parametrize("fuse", [replay.FUSE_NONE, replay.FUSE_REFERENCE])
def test_reference_single_conv(tmp_path, fuse):
    # the fused symbol is hard-wired to cuDNN's IMPLICIT_PRECOMP_GEMM, which needs a workspace
    (y,) = reference_outputs(tmp_path, "single_conv", fuse=fuse, workspace=32 << 20)
    (want,) = oracle_outputs("single_conv", 1, 0)
    assert max_rel_err(y, want) <= FP32_TOL


def test_reference_resnet50_unfused(tmp_path):
    """The configuration the reference's own scripts compile: no fusion, dealloc-opt, pool.
    Logits only: with random weights they reach the thousands, where the reference's softmax
    (global maximum found by a racy kernel, cuda/CUDASoftmaxFunc.cu:56-65) overflows."""
    (y,) = reference_outputs(tmp_path, "resnet50", 2, 64)
    (want,) = oracle_outputs("resnet50", 2, 64)
    assert max_rel_err(y, want) <= FP32_TOL
    assert np.array_equal(y.argmax(1), want.argmax(1))


def test_reference_mobilenet_v2_unfused(tmp_path):
    """DNNConvFunc with groups = C, DNNTensorOpFunc bias add and CUDAClipFunc, 17 times over
    (cudnn/CUDNNConvFunc.cpp:48-82, cuda/CUDAClipFunc.cu:5-28)."""
    (y,) = reference_outputs(tmp_path, "mobilenet_v2", 2, 96)
    (want,) = oracle_outputs("mobilenet_v2", 2, 96)
    assert max_rel_err(y, want) <= FP32_TOL
    assert np.array_equal(y.argmax(1), want.argmax(1))


def test_reference_vgg16_unfused(tmp_path):
    """Thirteen 3x3 convolutions, max pools, the 1x1 average pool, Flatten in NCHW order and
    the three-layer FC stack through cuBLASLt."""
    (y,) = reference_outputs(tmp_path, "vgg16", 2, 64)
    (want,) = oracle_outputs("vgg16", 2, 64)
    assert max_rel_err(y, want) <= FP32_TOL
    assert np.array_equal(y.argmax(1), want.argmax(1))


def test_reference_padded_average_pool(tmp_path):
    """Average pooling whose windows overhang the image: the reference's descriptor counts
    the padding in the divisor (cudnn/CUDNNAveragePoolFunc.cpp:43-60), and so does the oracle
    in the mode the runtime is compared with."""
    (y,) = reference_outputs(tmp_path, "avgpool_padded", 2, 9)
    (want,) = oracle_outputs("avgpool_padded", 2, 9)
    assert max_rel_err(y, want) <= FP32_TOL


def test_reference_depthwise_bias_clip(tmp_path):
    (y,) = reference_outputs(tmp_path, "depthwise_clip", 2, 15)
    (want,) = oracle_outputs("depthwise_clip", 2, 15)
    assert max_rel_err(y, want) <= FP32_TOL


def test_reference_gemm_softmax(tmp_path):
    """CUBLASMatmul2dFunc + bias add + CUDASoftmaxFunc on logits of ordinary magnitude (the
    reference's softmax is sound there)."""
    (y,) = reference_outputs(tmp_path, "softmax_head", 8, 1)
    (want,) = oracle_outputs("softmax_head", 8, 1)
    assert max_rel_err(y, want) <= FP32_TOL
    assert np.array_equal(y.argmax(1), want.argmax(1))
    np.testing.assert_allclose(y.sum(1), 1.0, rtol=1e-5)
