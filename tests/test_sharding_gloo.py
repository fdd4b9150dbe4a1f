"""The N > 1 path on CPU: two gloo ranks shard a batch, each evaluates its shard (with the
CPU oracle standing in for the GPU runtime), and the gathered logits equal the whole-batch
result in image order."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, batch, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from helpers import run_graph_oracle
    from occamy_b200 import graphs, sharding
    lo, hi = sharding.shard_range(batch, rank, world)
    g_full = graphs.resnet50(batch=batch, seed=0, softmax=False, image=32, num_classes=10)
    x = graphs.make_input(g_full, 0)
    g = graphs.resnet50(batch=hi - lo, seed=0, softmax=False, image=32, num_classes=10)
    (y,) = run_graph_oracle(g, x[lo:hi])
    out = sharding.gather_logits(torch.from_numpy(y))
    if rank == 0:
        (want,) = run_graph_oracle(g_full, x)
        q.put((out.numpy(), want))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_shard_and_gather():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + os.getpid() % 300
    procs = [ctx.Process(target=_worker, args=(r, 2, port, 4, q)) for r in range(2)]
    for p in procs:
        p.start()
    got, want = q.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert got.shape == want.shape == (4, 10)
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5)


def test_shard_range_rules():
    from occamy_b200 import sharding
    assert [sharding.shard_range(256, r, 8) for r in (0, 7)] == [(0, 32), (224, 256)]
    with pytest.raises(ValueError):
        sharding.shard_range(10, 0, 4)
    with pytest.raises(ValueError):
        sharding.shard_range(8, 8, 8)
