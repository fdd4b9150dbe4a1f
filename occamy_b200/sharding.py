"""Batch sharding of one inference over the ranks of a torch.distributed job.

Inference over independent images needs no exchange except at the end: rank r of R runs
images [r*B/R, (r+1)*B/R) with a full weight replica and its own pool plan, and the ranks'
logits are concatenated in rank order by one all-gather.  Backend-agnostic (NCCL on GPUs,
gloo in the CPU tests).
"""
from __future__ import annotations


def shard_range(batch: int, rank: int, world: int):
    """[start, stop) of the images rank `rank` owns; the batch must divide evenly so that
    every rank replays the same program shape."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    if batch % world:
        raise ValueError(f"global batch {batch} does not divide over {world} ranks")
    per = batch // world
    return rank * per, (rank + 1) * per


def gather_logits(local, out=None):
    """All-gather `local` ([B/R, classes] tensor) into [B, classes], rank order = image
    order.  Must be called by every rank of the default process group."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size() if dist.is_initialized() else 1
    if world == 1:
        if out is None:
            return local
        out.copy_(local)
        return out
    if out is None:
        out = torch.empty((local.shape[0] * world,) + tuple(local.shape[1:]), dtype=local.dtype,
                          device=local.device)
    dist.all_gather_into_tensor(out, local.contiguous())
    return out
