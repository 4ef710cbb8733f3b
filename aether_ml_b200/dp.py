"""Batch-sharded data parallelism for a :class:`aether_ml_b200.model.Model`: one process per GPU,
``torch.distributed`` (NCCL over NVLink on GPUs, gloo in the CPU tests) as plumbing, ONE all-reduce
of the flat gradient buffer per step.  The reference has no multi-GPU code; the sharding rule is

  * rank r of G takes samples [r*B/G, (r+1)*B/G) of every global batch;
  * each rank's loss gradient is already divided by its local sample count
    (CNN/models/CNN_classes_cupy.py:680), so the all-reduced SUM is turned into the global-batch
    gradient by the factor 1/G, folded into the Adam kernel (``Optimizer_Adam.grad_scale``);
  * parameters start identical (rank 0 broadcast) and stay bit-identical because every rank applies
    the same reduced gradient; Batch_Norm statistics stay per rank.
"""
import os

import torch
import torch.distributed as dist


def env_world():
    return int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))


def init_from_env(backend=None):
    """Join the process group described by RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT.
    Returns (world, rank, local_rank); a single process needs no group."""
    world, rank, local = env_world()
    if world > 1 and not dist.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        kwargs = {}
        if backend == "nccl":
            torch.cuda.set_device(local)
            kwargs["device_id"] = torch.device("cuda", local)
        dist.init_process_group(backend, **kwargs)
    elif torch.cuda.is_available():
        torch.cuda.set_device(local)
    return world, rank, local


def shard_bounds(n, rank, world):
    """[lo, hi) of the contiguous shard of `n` samples owned by `rank` (n must divide evenly so that
    every rank's local mean has the same weight in the average)."""
    if n % world:
        raise ValueError("global batch %d is not divisible by world size %d" % (n, world))
    per = n // world
    return rank * per, (rank + 1) * per


def shard_batch(X, y, rank, world):
    lo, hi = shard_bounds(len(X), rank, world)
    return X[lo:hi], y[lo:hi]


def allreduce_sum_(flat):
    """In-place sum of the flat gradient buffer over all ranks (no-op for a single process)."""
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(flat, op=dist.ReduceOp.SUM)
    return flat


def broadcast_(flat, src=0):
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.broadcast(flat, src=src)
    return flat


def attach(model):
    """Make a finalized model (``finalize(flat=True)``) data parallel: broadcast rank 0's parameters,
    all-reduce the flat gradient buffer before every optimizer step, average through grad_scale."""
    if model.flat_params is None:
        raise RuntimeError("data parallelism needs Model.finalize(flat=True)")
    world = dist.get_world_size() if dist.is_initialized() else 1
    broadcast_(model.flat_params)
    model.grad_hook = allreduce_sum_
    model.optimizer.grad_scale = 1.0 / world
    return world
