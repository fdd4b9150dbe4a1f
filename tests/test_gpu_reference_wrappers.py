"""Pins the CPU oracle against the reference's own runtime: the cuDNN / cuBLASLt wrappers of
corelab-src/occamy, compiled unchanged into oracle/_ref/ by oracle/build.py, replayed with
the same call programs.  Skipped when that library was not built.

cuDNN's default math mode may use TF32 tensor cores for fp32 convolutions on this GPU, so
the reference's outputs are compared with a 5e-3 bound rather than the 1e-4 of our fp32 mode.
"""
import os

import numpy as np
import pytest

from helpers import max_rel_err, run_graph_oracle
from occamy_b200 import graphs, replay
from oracle import build as obuild

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref_binding():
    if not os.path.exists(obuild.REF_SO):
        pytest.skip("reference wrappers not built (oracle/_ref)")
    try:
        return replay.Binding(obuild.REF_SO)
    except RuntimeError as e:
        pytest.skip(f"reference wrappers do not load here: {e}")


@pytest.mark.parametrize("fuse", [replay.FUSE_NONE, replay.FUSE_REFERENCE])
def test_reference_single_conv(ref_binding, fuse):
    g = graphs.single_conv(seed=0)
    x = graphs.make_input(g, 0, "uniform")
    p = g.to_program()
    # the fused symbol is hard-wired to cuDNN's IMPLICIT_PRECOMP_GEMM, which needs a workspace
    p.lower(fuse=fuse, workspace_bytes=32 << 20)
    (y,) = p.run(ref_binding, x)
    (want,) = run_graph_oracle(g, x)
    assert max_rel_err(y, want) <= 5e-3


def test_reference_resnet50_unfused(ref_binding):
    """The configuration the reference's own scripts compile: no fusion, dealloc-opt, pool.
    Logits only: with random weights they reach the thousands, where the reference's softmax
    (global maximum found by a racy kernel, cuda/CUDASoftmaxFunc.cu:56-65) overflows."""
    g = graphs.resnet50(batch=2, seed=0, softmax=False, image=64)
    x = graphs.make_input(g, 0)
    p = g.to_program()
    p.lower(fuse=replay.FUSE_NONE, workspace_bytes=1 << 20)
    (y,) = p.run(ref_binding, x)
    (want,) = run_graph_oracle(g, x)
    assert max_rel_err(y, want) <= 5e-3
    assert np.array_equal(y.argmax(1), want.argmax(1))
