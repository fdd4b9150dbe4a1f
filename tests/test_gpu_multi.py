"""Batch sharding on real GPUs: two ranks, each with half of the batch, logits gathered with
NCCL, compared with the CPU oracle on images of BOTH shards (`bench.py`'s own parity check on
the gathered tensor).  Needs two GPUs; skipped on a single-GPU box.  The launch is the one the
benchmark is run with: one process per GPU under torch.distributed.run, rendezvous on 127.0.0.1.
"""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_two_ranks_gathered_logits_match_the_oracle(native_libs):
    torch = pytest.importorskip("torch")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29533", os.path.join(ROOT, "bench.py"),
           "--gpus", "2", "--batch", "64", "--steps", "3", "--warmup", "3", "--warm-seconds", "0",
           "--no-extras", "--no-cpu-baseline"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads([ln for ln in r.stdout.splitlines() if ln.startswith("{")][-1])
    assert line["n_gpus"] == 2 and line["config"]["global_batch"] == 64
    p = line["parity_checked"]
    # rows 0.. belong to rank 0, the last two to rank 1
    assert p["ok"] and p["top1_equal"] and p["max_rel"] <= 2e-2
    assert max(p["rows"]) >= 32
