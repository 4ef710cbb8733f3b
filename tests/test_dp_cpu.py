"""CPU tests (gloo, world_size 2) of the data-parallel plumbing: contiguous batch shards, one summed
all-reduce of a flat gradient buffer, 1/G averaging -- checked against the NumPy oracle: the average
of the per-shard gradients of a conv + dense stack equals the gradient of the whole batch."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _oracle_grads(x, labels, w, wd):
    """Mean-loss gradients of conv(3x3 same) -> flatten -> dense -> softmax/CCE on one shard."""
    from oracle import aether_oracle as O
    y = O.conv_forward(x, w, np.zeros(w.shape[3]))
    flat = y.reshape(len(x), -1)
    z = O.dense_forward(flat, wd, np.zeros((1, wd.shape[1])))
    dz = O.softmax_cce_backward(O.softmax(z), labels, 0.01)
    dflat, dwd, _ = O.dense_backward(flat, wd, np.zeros((1, wd.shape[1])), dz)
    _, dw, db = O.conv_backward(x, w, dflat.reshape(y.shape))
    return np.concatenate([dw.ravel(), db.ravel(), dwd.ravel()])


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    from aether_ml_b200 import dp
    w_, r_, _ = dp.init_from_env("gloo")
    assert (w_, r_) == (world, rank)
    rng = np.random.default_rng(0)                       # same data on every rank; each takes its shard
    X = rng.random((8, 6, 6, 3)); labels = rng.integers(0, 5, 8)
    w = rng.standard_normal((3, 3, 3, 4)) * 0.3; wd = rng.standard_normal((6 * 6 * 4, 5)) * 0.1
    xs, ys = dp.shard_batch(X, labels, rank, world)
    assert len(xs) == 4 and np.array_equal(xs, X[rank * 4:(rank + 1) * 4])
    flat = torch.from_numpy(_oracle_grads(xs, ys, w, wd))
    dp.allreduce_sum_(flat)
    avg = flat.numpy() / world
    full = _oracle_grads(X, labels, w, wd)
    # the same gradients reduced in buckets: bucket order = backward order (tail of the buffer first), each bucket
    # reduced once, the result equal to the single all-reduce
    n_conv = w.size + w.shape[3]
    ranges = [(0, n_conv), (n_conv, n_conv + wd.size)]   # conv layer, dense layer (forward order)
    buckets = dp.plan_buckets(ranges, 2)
    assert buckets == [(n_conv, n_conv + wd.size, 1), (0, n_conv, 0)]
    assert dp.plan_buckets(ranges, 1) == [(0, n_conv + wd.size, 0)]
    assert dp.plan_buckets(ranges, 5) == buckets                      # never more buckets than layers
    flat_b = torch.from_numpy(_oracle_grads(xs, ys, w, wd))
    red = dp.BucketReducer(flat_b, buckets)
    assert red.active
    red.start(0)                                         # the dense head is complete first ...
    head_before_wait = flat_b[:n_conv].clone()           # ... while the conv part is still this rank's own gradient
    red.wait(0)
    assert torch.equal(flat_b[:n_conv], head_before_wait)
    assert torch.allclose(flat_b[n_conv:], flat[n_conv:], rtol=0, atol=0)
    red.start(1)
    red.wait(1)
    assert torch.equal(flat_b, flat)
    flat_c = torch.from_numpy(_oracle_grads(xs, ys, w, wd))
    assert torch.equal(dp.BucketReducer(flat_c, buckets).reduce_all(), flat)
    params = torch.full((5,), float(rank))
    dp.broadcast_(params)
    if rank == 0:
        out.put((float(np.abs(avg - full).max() / np.abs(full).max()), params.tolist()))
    else:
        assert params.tolist() == [0.0] * 5
    torch.distributed.destroy_process_group()


def test_two_rank_gradient_average_matches_full_batch():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    hung = [p for p in procs if p.exitcode is None]
    for p in hung:                       # never leave a worker behind in a half-finished collective
        p.kill()
        p.join(10)
    assert not hung, "a data-parallel worker did not finish"
    assert all(p.exitcode == 0 for p in procs)
    err, params = out.get(timeout=10)
    assert err < 1e-12
    assert params == [0.0] * 5


def test_shard_bounds():
    from aether_ml_b200 import dp
    assert [dp.shard_bounds(4096, r, 8) for r in (0, 7)] == [(0, 512), (3584, 4096)]
    with pytest.raises(ValueError):
        dp.shard_bounds(10, 0, 4)
    assert dp.env_world()[0] >= 1
