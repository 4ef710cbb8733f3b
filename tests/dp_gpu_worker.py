"""Worker of tests/test_dp_gpu.py, run once per GPU under torch.distributed.run: the data-parallel train step on
real GPUs over NCCL.  Checks, on every rank:
  * the bucket-reduced gradient buffer equals the all-gathered sum of the ranks' own gradients;
  * the step captured as ONE graph with the bucketed all-reduces inside replays to the same parameters as eager
    steps with a single all-reduce after the whole backward;
  * the parameters stay identical on all ranks.
Prints "DP_GPU_OK <world>" from rank 0 when everything held."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from aether_ml_b200 import dp, layers as Ly  # noqa: E402
from aether_ml_b200.model import Accuracy_Categorical, Model  # noqa: E402


def build(buckets):
    np.random.seed(5)                                    # same initial parameters on every rank
    m = Model()
    c_in, hw = 3, 16
    for c_out in (32, 64):
        m.add(Ly.Conv_Layer((hw, hw, c_in), c_out, (3, 3), (1, 1), "same", math_mode="bf16"))
        m.add(Ly.Batch_Norm(n_features=c_out))
        m.add(Ly.ReLU())
        m.add(Ly.Pooling((2, 2), (2, 2), "valid", "max"))
        c_in, hw = c_out, hw // 2
    m.add(Ly.Flatten())
    m.add(Ly.Layer_Dense(4 * 4 * 64, 128, weight_regularizer_l2=2e-5, math_mode="bf16"))
    m.add(Ly.Leaky_ReLU(0.01))
    m.add(Ly.Layer_Dense(128, 10, math_mode="bf16"))
    m.add(Ly.SoftMax())
    m.set(loss=Ly.Loss_CategoricalCrossEntropy(label_smoothing=0.01), optimizer=Ly.Optimizer_Adam(learning_rate=1e-3, decay=5e-5),
          accuracy=Accuracy_Categorical())
    m.finalize(flat=True, fuse=True)
    dp.attach(m, buckets=buckets)
    return m


def note(rank, what):
    print("[dp_gpu_worker rank %d] %s" % (rank, what), file=sys.stderr, flush=True)


def rel(a, b):
    return float((a.double() - b.double()).norm() / b.double().norm())


def main():
    world, rank, local = dp.init_from_env(timeout_s=int(os.environ.get("AETHER_DP_TIMEOUT_S", "60")))
    assert world >= 2
    rng = np.random.default_rng(3)                       # the same global batches everywhere; each rank takes its shard
    batches = []
    for _ in range(4):
        X = rng.random((16 * world, 16, 16, 3)).astype(np.float32)
        y = rng.integers(0, 10, 16 * world)
        batches.append(dp.shard_batch(X, y, rank, world))

    bucketed, single = build(2), build(1)
    single.enable_device_step()                          # Adam's step count on the device in both, as under capture
    assert len(bucketed.bucket_reducer.buckets) == 2 and len(single.bucket_reducer.buckets) == 1
    assert bucketed.bucket_reducer.active

    note(rank, "models built")
    # 1. reduced buffer == all-gathered sum
    held, bucketed._bucket_of_layer = bucketed._bucket_of_layer, {}
    out = bucketed.forward(batches[0][0], training=True)
    bucketed.backward(out, batches[0][1])
    bucketed._bucket_of_layer = held
    own = bucketed.flat_grads.clone()
    gathered = [torch.empty_like(own) for _ in range(world)]
    dist.all_gather(gathered, own)
    want = torch.stack(gathered).double().sum(dim=0)
    bucketed.bucket_reducer.reduce_all()
    assert rel(bucketed.flat_grads, want) <= 1e-6
    assert rel(own, want) > 0.05                         # one rank's gradient is not the sum

    note(rank, "reduced buffer checked")
    # 2. one captured graph with the collectives inside == eager steps with one all-reduce
    bucketed.capture_train_step(*batches[0])
    note(rank, "captured: " + bucketed.capture_note)
    assert "all-reduce bucket" in bucketed.capture_note, bucketed.capture_note
    for X, y in batches:
        bucketed.train_step_graph(X, y)
        single.train_step(X, y)
    torch.cuda.synchronize()
    assert rel(bucketed.flat_params, single.flat_params) <= 1e-6, rel(bucketed.flat_params, single.flat_params)

    note(rank, "graph steps == eager steps")
    # 3. identical parameters on all ranks
    mine = bucketed.flat_params.clone()
    theirs = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(theirs, mine)
    assert all(torch.equal(t, mine) for t in theirs)

    note(rank, "parameters identical on all ranks")
    # 4. the fallback form (collectives launched eagerly between two graphs) gives the same parameters
    fallback = build(2)
    fallback.capture_train_step(*batches[0], collectives_in_graph=False)
    note(rank, "captured: " + fallback.capture_note)
    assert fallback.capture_note.startswith("two graphs")
    for X, y in batches:
        fallback.train_step_graph(X, y)
    torch.cuda.synchronize()
    assert rel(fallback.flat_params, single.flat_params) <= 1e-6

    note(rank, "fallback steps == eager steps")
    dist.barrier()
    if rank == 0:
        print("DP_GPU_OK %d" % world, flush=True)
    dp.shutdown(bucketed, single, fallback)              # graphs first, then the process group
    note(rank, "process group destroyed")


if __name__ == "__main__":
    main()
