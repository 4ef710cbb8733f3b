"""Batch-sharded data parallelism for a :class:`aether_ml_b200.model.Model`: one process per GPU,
``torch.distributed`` (NCCL over NVLink on GPUs, gloo in the CPU tests) as plumbing.  The reference has no
multi-GPU code; the sharding rule is

  * rank r of G takes samples [r*B/G, (r+1)*B/G) of every global batch;
  * each rank's loss gradient is already divided by its local sample count
    (CNN/models/CNN_classes_cupy.py:680), so the all-reduced SUM is turned into the global-batch
    gradient by the factor 1/G, folded into the Adam kernel (``Optimizer_Adam.grad_scale``);
  * parameters start identical (rank 0 broadcast) and stay bit-identical because every rank applies
    the same reduced gradient; Batch_Norm statistics stay per rank.

The flat gradient buffer is reduced in buckets, in the order the backward pass finishes them: the layers
nearest the loss (the dense head, most of the bytes in the reference's CNNs) are complete first, so their
all-reduce is started on NCCL's own stream while the convolution blocks are still back-propagating; each
bucket's Adam update waits only for its own all-reduce.  ``buckets=1`` gives the single all-reduce after
the whole backward.
"""
import datetime
import os

import torch
import torch.distributed as dist


def env_world():
    return int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))


def init_from_env(backend=None, timeout_s=None):
    """Join the process group described by RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT.
    Returns (world, rank, local_rank); a single process needs no group.  Collectives give up after
    ``timeout_s`` seconds ($AETHER_DP_TIMEOUT_S, default 300) with an error instead of waiting for a rank
    that will never arrive."""
    world, rank, local = env_world()
    if world > 1 and not dist.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        if timeout_s is None:
            timeout_s = int(os.environ.get("AETHER_DP_TIMEOUT_S", "300"))
        kwargs = {"timeout": datetime.timedelta(seconds=timeout_s)}
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


def plan_buckets(layer_ranges, n_buckets=2):
    """Splits the flat gradient buffer into at most ``n_buckets`` contiguous buckets at layer boundaries.

    ``layer_ranges`` lists (lo, hi) element ranges of the trainable layers in FORWARD order (contiguous,
    ascending).  The backward pass completes them last to first, so the buckets are returned in that order:
    the first bucket is the tail of the buffer.  Each bucket is ``(lo, hi, trigger)`` where ``trigger`` is the
    index (into ``layer_ranges``) of the layer whose backward completes the bucket, i.e. its first layer in
    forward order.  Boundaries are chosen greedily so every bucket but the last holds at least 1/n_buckets of
    the elements: for the reference's CNNs the dense head alone fills the first bucket."""
    n = len(layer_ranges)
    if n == 0:
        return []
    total = layer_ranges[-1][1] - layer_ranges[0][0]
    want = max(1, int(n_buckets))
    buckets, hi_layer, acc = [], n, 0
    for k in range(n - 1, -1, -1):
        acc += layer_ranges[k][1] - layer_ranges[k][0]
        last = len(buckets) == want - 1
        if (not last and acc * want >= total) or k == 0:
            buckets.append((layer_ranges[k][0], layer_ranges[hi_layer - 1][1], k))
            hi_layer, acc = k, 0
            if k == 0:
                break
    return buckets


class BucketReducer:
    """All-reduces ``flat[lo:hi]`` bucket by bucket.  ``start(i)`` launches bucket i's all-reduce without
    waiting for it (on GPUs it runs on NCCL's stream behind what the calling stream has queued so far);
    ``wait(i)`` makes the calling stream wait for it.  Works on any tensor ``torch.distributed`` accepts,
    so the bookkeeping is testable with gloo on CPU tensors."""

    def __init__(self, flat, buckets):
        self.flat = flat
        self.buckets = list(buckets)
        self.works = [None] * len(self.buckets)
        self.active = dist.is_initialized() and dist.get_world_size() > 1

    def start(self, i):
        if not self.active:
            return
        lo, hi, _ = self.buckets[i]
        self.works[i] = dist.all_reduce(self.flat[lo:hi], op=dist.ReduceOp.SUM, async_op=True)

    def wait(self, i):
        w = self.works[i]
        if w is not None:
            w.wait()
            self.works[i] = None

    def reduce_all(self):
        for i in range(len(self.buckets)):
            self.start(i)
        for i in range(len(self.buckets)):
            self.wait(i)
        return self.flat


def attach(model, buckets=2):
    """Make a finalized model (``finalize(flat=True)``) data parallel: broadcast rank 0's parameters, reduce the
    flat gradient buffer in ``buckets`` buckets as the backward pass completes them, average through
    grad_scale.  Returns the world size."""
    if model.flat_params is None:
        raise RuntimeError("data parallelism needs Model.finalize(flat=True)")
    world = dist.get_world_size() if dist.is_initialized() else 1
    broadcast_(model.flat_params)
    model.optimizer.grad_scale = 1.0 / world
    model.grad_hook = None
    model.set_bucket_reducer(BucketReducer(model.flat_grads, plan_buckets(model.flat_layer_ranges, buckets)))
    return world


def shutdown(*models):
    """Ends data-parallel work: releases the models' captured graphs first (a graph that recorded collectives pins
    the NCCL communicator, and ``destroy_process_group`` then never returns), then destroys the process group."""
    import gc
    for m in models:
        m.release_graphs()
    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    if dist.is_initialized():
        dist.destroy_process_group()
