"""GPU test of a whole training step through Model (conv blocks + dense head + Adam) against the
same network evaluated with the NumPy oracle, for the two network topologies of the reference's
example scripts (Fashion-MNIST-shaped and CIFAR-shaped, scaled down in batch)."""
import os
import pickle

import numpy as np
import pytest

from oracle import aether_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    import torch
    from aether_ml_b200 import _lib, layers, model
    if not torch.cuda.is_available():
        pytest.fail("CUDA device required for -m gpu tests")
    return torch, _lib, layers, model


def host(t):
    return t.detach().cpu().numpy().astype(np.float64)


def build(env, topology, mode, flat, fuse=False):
    torch, _lib, Ly, M = env
    np.random.seed(42)
    m = M.Model()
    if topology == "fmnist":           # Conv 1->32, BN, ReLU, Pool, Conv 32->64, BN, ReLU, Pool, Flatten, Dense, Dense, SoftMax
        shape, chans, dense = (28, 28, 1), (32, 64), (7 * 7 * 64, 128)
        drop_sp, drop = (None, None), None
    else:                              # CIFAR-shaped 3-block CNN with spatial dropout, LeakyReLU dense, dropout
        shape, chans, dense = (32, 32, 3), (32, 64, 128), (4 * 4 * 128, 256)
        drop_sp, drop = (0.075, 0.1, None), 0.075
    h, w, c = shape
    for k, co in enumerate(chans):
        m.add(Ly.Conv_Layer((h, w, c), co, (3, 3), (1, 1), "same", math_mode=mode))
        m.add(Ly.Batch_Norm(n_features=co))
        m.add(Ly.ReLU())
        if topology == "cifar" and drop_sp[k]:
            m.add(Ly.Layer_Dropout_Spatial(drop_sp[k]))
        m.add(Ly.Pooling((2, 2), (2, 2), "valid", "max"))
        h, w, c = h // 2, w // 2, co
    m.add(Ly.Flatten())
    if topology == "cifar":
        m.add(Ly.Layer_Dense(dense[0], dense[1], weight_regularizer_l2=2e-5, math_mode=mode))
        m.add(Ly.Leaky_ReLU(0.01))
        m.add(Ly.Layer_Dropout(drop, seed=77))
    else:
        m.add(Ly.Layer_Dense(dense[0], dense[1], math_mode=mode))
    m.add(Ly.Layer_Dense(dense[1], 10, math_mode=mode))
    m.add(Ly.SoftMax())
    m.set(loss=Ly.Loss_CategoricalCrossEntropy(label_smoothing=0.01),
          optimizer=Ly.Optimizer_Adam(learning_rate=1e-3, decay=5e-5), accuracy=M.Accuracy_Categorical())
    m.finalize(flat=flat, fuse=fuse)
    return m, shape


def oracle_step(m, Ly, X, y):
    """Replays forward/backward of the device model's layer list with the NumPy oracle, reading the
    parameters (and the dropout masks the device drew) from the device layers.  Returns
    (probabilities, {layer index: (dw, db)})."""
    acts, ctx = [np.asarray(X, np.float64)], []
    for l in m.layers:
        a = acts[-1]
        n = type(l).__name__
        if n == "Conv_Layer":
            out = O.conv_forward(a, host(l.weights), host(l.biases)); ctx.append(None)
        elif n == "Batch_Norm":
            C = a.shape[-1]
            out, _, mean, var, _, _ = O.bn_forward_train(a, host(l.gamma), host(l.beta), np.zeros(C), np.ones(C)); ctx.append((mean, var))
        elif n == "ReLU":
            out = O.relu_forward(a); ctx.append(None)
        elif n == "Leaky_ReLU":
            out = O.leaky_relu_forward(a, l.alpha); ctx.append(None)
        elif n == "Layer_Dropout_Spatial":
            mask = host(l.channel_mask); out = a * mask; ctx.append(mask)
        elif n == "Layer_Dropout":
            mask = host(l.binary_mask); out = a * mask; ctx.append(mask)
        elif n == "Pooling":
            out, arg = O.pool_forward(a); ctx.append(arg)
        elif n == "Flatten":
            out = a.reshape(len(a), -1); ctx.append(a.shape)
        elif n == "Layer_Dense":
            out = O.dense_forward(a, host(l.weights), host(l.biases)); ctx.append(None)
        elif n == "SoftMax":
            out = O.softmax(a); ctx.append(None)
        acts.append(out)
    probs = acts[-1]
    g = O.softmax_cce_backward(probs, y, 0.01)
    grads = {}
    for k in range(len(m.layers) - 2, -1, -1):
        l, a, n = m.layers[k], acts[k], type(m.layers[k]).__name__
        if n == "Conv_Layer":
            g, dw, db = O.conv_backward(a, host(l.weights), g); grads[k] = (dw, db)
        elif n == "Batch_Norm":
            g, dg, dbeta = O.bn_backward(a, g, host(l.gamma), *ctx[k]); grads[k] = (dg, dbeta)
        elif n == "ReLU":
            g = O.relu_backward(a, g)
        elif n == "Leaky_ReLU":
            g = O.leaky_relu_backward(a, g, l.alpha)
        elif n in ("Layer_Dropout_Spatial", "Layer_Dropout"):
            g = g * ctx[k]
        elif n == "Pooling":
            g = O.pool_backward(g, a.shape, ctx[k])
        elif n == "Flatten":
            g = g.reshape(ctx[k])
        elif n == "Layer_Dense":
            g, dw, db = O.dense_backward(a, host(l.weights), host(l.biases), g, wl2=l.weight_regularizer_l2); grads[k] = (dw, db)
    return probs, grads


@pytest.mark.parametrize("topology,mode,flat,tol", [("fmnist", "tf32", False, 4e-3), ("cifar", "bf16", True, 4e-2),
                                                   ("cifar", "fp32", False, 1e-4)])
def test_train_step_matches_oracle(env, topology, mode, flat, tol):
    torch, _lib, Ly, M = env
    m, shape = build(env, topology, mode, flat)
    rng = np.random.default_rng(9)
    S = 16
    X = rng.random((S,) + shape).astype(np.float32)
    y = rng.integers(0, 10, S)
    # randomise BN affine parameters and biases so every gradient path is exercised
    for l in m.trainable_layers:
        l.biases.copy_(torch.from_numpy((rng.standard_normal(tuple(l.biases.shape)) * 0.1).astype(np.float32)))
    before = [(host(l.weights).copy(), host(l.biases).copy()) for l in m.trainable_layers]
    m.loss.new_pass()
    out = m.forward(X, training=True)
    data_loss, reg_loss = m.loss.calculate(out, y, include_regularization=True, training=True)
    probs_o, grads_o = oracle_step(m, Ly, X, y)
    m.backward(out, y)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert O.rel_l2(host(out), probs_o) <= tol
    assert abs(float(data_loss) - O.cce_loss(probs_o, y, 0.01, True).mean()) <= tol * 3
    # errors compound through the depth of the network: the tolerance is per network, not per layer
    for k, (dw, db) in grads_o.items():
        l = m.layers[k]
        # Batch_Norm's dgamma = sum(dy * xhat) cancels heavily as well, hence the wider factor there
        wfac = 10 if type(l).__name__ == "Batch_Norm" else 5
        assert O.rel_l2(host(l.dweights), dw) <= tol * wfac, (k, type(l).__name__)
        # bias gradients are sums with heavy cancellation (exactly zero for a bias that feeds a Batch_Norm, whose
        # batch mean is subtracted again): judge them on the scale of the layer's weight gradient when that is larger
        dbd = host(l.dbiases).reshape(db.shape)
        scale = max(np.linalg.norm(db), np.linalg.norm(dw))
        assert np.linalg.norm(dbd - db) <= tol * 5 * scale, (k, type(l).__name__)
    if topology == "cifar":
        first_dense = next(l for l in m.layers if type(l).__name__ == "Layer_Dense")
        w0 = before[m.trainable_layers.index(first_dense)][0]
        assert np.isclose(float(reg_loss), 2e-5 * (w0 ** 2).sum(), rtol=1e-4)
    # optimizer: replay Adam on the DEVICE gradients so only the update rule is compared
    dev_grads = [(host(l.dweights).copy(), host(l.dbiases).copy()) for l in m.trainable_layers]
    m._apply_optimizer()
    for (w0, b0), (gw, gb), l in zip(before, dev_grads, m.trainable_layers):
        w1, _, _ = O.adam_step(w0, gw, 0, 0, 1e-3, 0)
        b1, _, _ = O.adam_step(b0, gb.reshape(b0.shape), 0, 0, 1e-3, 0)
        assert O.rel_l2(host(l.weights), w1) <= 1e-5 and O.rel_l2(host(l.biases), b1) <= 1e-4
    assert m.optimizer.iterations == 1


def test_train_loop_evaluate_predict_save_load(env, tmp_path, capsys):
    torch, _lib, Ly, M = env
    m, shape = build(env, "fmnist", "bf16", True)
    rng = np.random.default_rng(3)
    y = rng.integers(0, 2, 64)                                                            # separable 2-class data:
    X = (rng.random((64,) + shape) * 0.3 + 0.7 * y[:, None, None, None]).astype(np.float32)   # dark vs bright images
    m.train(X, y, epochs=20, batch_size=32, print_every=100, validation_data=(X, y))
    printed = capsys.readouterr().out
    assert "Training" in printed and "Valdiation" in printed
    acc, loss = m.evaluate(X, y, batch_size=32)
    assert acc > 0.9 and np.isfinite(loss)
    pred = m.predict(X, batch_size=16)
    assert tuple(pred.shape) == (64, 10)
    path = os.path.join(tmp_path, "params")
    m.save_parameters(path)
    saved = pickle.load(open(path, "rb"))
    assert len(saved) == len(m.trainable_layers) and saved[0][0].shape == (3, 3, 1, 32) and saved[1][2].shape == (1, 1, 1, 32)
    m2, _ = build(env, "fmnist", "bf16", False)
    m2.load_parameters(path)
    assert O.rel_l2(host(m2.predict(X, batch_size=16)), host(pred)) <= 1e-6
    conv = m2.layers[0]
    assert conv.weights is conv.filter_weights


@pytest.mark.parametrize("hook", [False, True])
def test_train_step_cuda_graph_matches_eager(env, hook):
    """A train step captured in a CUDA graph (Model.capture_train_step) replays to the same parameters as the
    eager steps: Adam's iteration count / decayed learning rate and the dropout draws come from a device counter,
    so every replay is a NEW step, and capturing itself does not train."""
    torch, _lib, Ly, M = env
    rng = np.random.default_rng(9)
    batches = [((rng.random((16, 32, 32, 3))).astype(np.float32), rng.integers(0, 10, 16)) for _ in range(4)]

    def fresh():
        m, _ = build(env, "cifar", "bf16", True)
        for k, l in enumerate(m.layers):                   # identical dropout streams in both models
            if hasattr(l, "seed"):
                l.seed = 1000 + k
        if hook:                                           # a gradient hook (the data-parallel all-reduce in real use)
            m.grad_hook = lambda g: g.mul_(0.5)            # runs eagerly between the two captured graphs
        return m

    eager = fresh()
    eager.enable_device_step()
    for X, y in batches:
        eager.train_step(X, y)
    masks_eager = [host(l.channel_mask) for l in eager.layers if isinstance(l, Ly.Layer_Dropout_Spatial)]

    graph = fresh()
    p0 = host(graph.flat_params).copy()
    graph.capture_train_step(*batches[0])
    assert np.array_equal(host(graph.flat_params), p0) and graph.optimizer.iterations == 0
    outs = []
    for X, y in batches:
        outs.append(host(graph.train_step_graph(X, y)).copy())
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert graph.optimizer.iterations == len(batches) == int(graph._g_step.item())
    assert O.rel_l2(host(graph.flat_params), host(eager.flat_params)) <= 1e-6
    assert O.rel_l2(host(graph.flat_m), host(eager.flat_m)) <= 1e-6
    assert not np.allclose(outs[0], outs[1])               # a replay sees the new batch and the new parameters
    masks_graph = [host(l.channel_mask) for l in graph.layers if isinstance(l, Ly.Layer_Dropout_Spatial)]
    for a, b in zip(masks_eager, masks_graph):
        assert np.array_equal(a, b)
    # the element dropout drew a different mask in every step (the device counter moved)
    drop = [l for l in graph.layers if isinstance(l, Ly.Layer_Dropout)][0]
    m_last = host(drop.binary_mask).copy()
    graph.train_step_graph(*batches[0])
    assert not np.array_equal(host(drop.binary_mask), m_last)
    assert abs((m_last > 0).mean() - (1 - 0.075)) < 0.05


@pytest.mark.parametrize("topology", ["fmnist", "cifar"])
def test_fused_batch_norm_activation_matches_unfused(env, topology):
    """finalize(fuse=True): the ReLU behind every Batch_Norm is applied inside the Batch_Norm kernels (forward,
    backward, inference), a spatial-dropout mask behind it is folded into the Batch_Norm coefficients and a 2x2
    pooling behind those is reduced in the same pass (the Batch_Norm then outputs the pooled tensor).  Same
    parameters after training steps and same predictions as the layer-by-layer model, up to the noise of the
    different summation order: a convolution bias in front of a Batch_Norm has a gradient that is zero in exact
    arithmetic, Adam turns its rounding noise into steps of the size of the learning rate, and a last-bit difference
    can flip a bf16 rounding in the next convolution."""
    torch, _lib, Ly, M = env
    rng = np.random.default_rng(21)
    tol = 5e-3
    plain, shape = build(env, topology, "bf16", True, fuse=False)
    fused, _ = build(env, topology, "bf16", True, fuse=True)
    for m in (plain, fused):
        m.enable_device_step()                             # identical dropout draws in both models
        for k, l in enumerate(m.layers):
            if hasattr(l, "seed"):
                l.seed = 500 + k
    assert any(getattr(l, "fused_into_prev", False) for l in fused.layers)
    assert not any(getattr(l, "fused_into_prev", False) for l in plain.layers)
    assert np.array_equal(host(plain.flat_params), host(fused.flat_params))
    for _ in range(3):
        X = rng.random((24,) + shape).astype(np.float32)
        y = rng.integers(0, 10, 24)
        op = plain.train_step(X, y)
        of = fused.train_step(X, y)
        assert O.rel_l2(host(of), host(op)) <= tol
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert O.rel_l2(host(fused.flat_params), host(plain.flat_params)) <= tol
    assert O.rel_l2(host(fused.flat_grads), host(plain.flat_grads)) <= 10 * tol
    Xe = rng.random((16,) + shape).astype(np.float32)
    assert O.rel_l2(host(fused.predict(Xe, batch_size=8)), host(plain.predict(Xe, batch_size=8))) <= tol
    drops = [l for l in fused.layers if isinstance(l, Ly.Layer_Dropout_Spatial)]
    assert all(d.fused_into_prev and d.output is d.inputs for d in drops)
    # the fused Batch_Norm exposes the ACTIVATED tensor and the ReLU hands it through
    bn = [l for l in fused.layers if isinstance(l, Ly.Batch_Norm)][0]
    act = bn.next
    assert act.output is bn.output and float(bn.output.min()) >= 0.0
    # ... and the pooling behind it is done by the same kernels: the Batch_Norm's output is the pooled tensor
    pool = [l for l in fused.layers if isinstance(l, Ly.Pooling)][0]
    assert bn.pooled_now and pool.output is bn.output and tuple(bn.output.shape[1:3]) == (shape[0] // 2, shape[1] // 2)


def _parse_lines(text):
    """(acc, loss, data_loss, reg_loss) of every 'epoch: ...' / ' training, ...' line Model.train printed."""
    import re
    rows = []
    for line in text.splitlines():
        m = re.search(r"acc: ([\d.]+), loss: ([\d.]+) \(data_loss: ([\d.]+), reg_loss: ([\d.]+)", line)
        if m:
            rows.append(tuple(float(v) for v in m.groups()))
    return rows


def test_train_loop_on_captured_step_prints_the_eager_numbers(env, capsys):
    """Model.train on the captured step (loss / accuracy accumulated on the device, read back only for printed
    lines) prints the same lines as the eager loop of the reference and ends with the same parameters."""
    torch, _lib, Ly, M = env
    rng = np.random.default_rng(31)
    y = rng.integers(0, 10, 96)
    X = rng.random((96, 32, 32, 3)).astype(np.float32)

    def run(use_graph):
        m, _ = build(env, "cifar", "bf16", True)
        m.enable_device_step()                             # the same dropout draws in both loops
        for k, l in enumerate(m.layers):
            if hasattr(l, "seed"):
                l.seed = 900 + k
        capsys.readouterr()
        m.train(X, y, epochs=2, batch_size=32, print_every=2, use_graph=use_graph)
        torch.cuda.synchronize()
        return m, capsys.readouterr().out

    eager, text_e = run(False)
    graph, text_g = run(True)
    assert graph._graph is not None and eager._graph is None
    rows_e, rows_g = _parse_lines(text_e), _parse_lines(text_g)
    assert len(rows_e) == len(rows_g) == 2 * 2 + 1          # steps 0 and 2 of each epoch + the closing line
    assert [l.split(",")[0] for l in text_e.splitlines()] == [l.split(",")[0] for l in text_g.splitlines()]
    for a, b in zip(rows_e, rows_g):
        assert np.allclose(a, b, atol=2e-3), (a, b)
    assert O.rel_l2(host(graph.flat_params), host(eager.flat_params)) <= 1e-5
    assert graph.optimizer.iterations == eager.optimizer.iterations == 6
    # ragged last batch: the loop falls back to the eager step by itself
    m3, _ = build(env, "cifar", "bf16", True)
    m3.train(X[:80], y[:80], epochs=1, batch_size=32, print_every=10)
    assert m3._graph is None


def test_gradient_buckets_follow_the_backward_order(env):
    """dp.plan_buckets on a real model: two buckets, the dense head first (it is complete first in the backward
    pass and holds most of the elements), the convolution blocks second; a single-process reducer changes nothing."""
    torch, _lib, Ly, M = env
    from aether_ml_b200 import dp
    m, shape = build(env, "cifar", "bf16", True)
    ranges = m.flat_layer_ranges
    assert ranges[0][0] == 0 and ranges[-1][1] == m.flat_params.numel()
    assert all(a[1] == b[0] for a, b in zip(ranges[:-1], ranges[1:]))
    buckets = dp.plan_buckets(ranges, 2)
    assert len(buckets) == 2
    (lo1, hi1, t1), (lo2, hi2, t2) = buckets
    assert hi1 == m.flat_params.numel() and lo1 == hi2 and lo2 == 0 and t2 == 0
    assert isinstance(m.trainable_layers[t1], Ly.Layer_Dense) and hi1 - lo1 > hi2 - lo2
    assert dp.plan_buckets(ranges, 1) == [(0, m.flat_params.numel(), 0)]
    ref, _ = build(env, "cifar", "bf16", True)
    dp.attach(m, buckets=2)
    assert m.bucket_reducer is not None and not m.bucket_reducer.active
    rng = np.random.default_rng(2)
    for mm in (m, ref):
        mm.enable_device_step()
        for k, l in enumerate(mm.layers):
            if hasattr(l, "seed"):
                l.seed = 40 + k
    for _ in range(2):
        X = rng.random((8,) + shape).astype(np.float32); y = rng.integers(0, 10, 8)
        m.train_step(X, y); ref.train_step(X, y)
    assert O.rel_l2(host(m.flat_params), host(ref.flat_params)) <= 1e-6      # per-bucket Adam == one Adam launch


def test_reference_checkpoint_file_loads_and_predicts(env, golden):
    """A parameter file in the reference CuPy model's format (pickled cupy arrays, float64 dense layers, keep-dims
    running statistics) loads through Model.load_parameters without CuPy and reproduces the probabilities the
    reference's NumPy model computed with those parameters."""
    torch, _lib, Ly, M = env
    g = golden("checkpoint_cupy_format")
    np.random.seed(1)
    m = M.Model()
    m.add(Ly.Conv_Layer((8, 8, 1), 4, (3, 3), (1, 1), "same"))
    m.add(Ly.Batch_Norm())
    m.add(Ly.ReLU())
    m.add(Ly.Pooling((2, 2), (2, 2), "valid", "max"))
    m.add(Ly.Conv_Layer((4, 4, 4), 8, (3, 3), (1, 1), "same"))
    m.add(Ly.Batch_Norm())
    m.add(Ly.ReLU())
    m.add(Ly.Pooling((2, 2), (2, 2), "valid", "max"))
    m.add(Ly.Flatten())
    m.add(Ly.Layer_Dense(2 * 2 * 8, 12))
    m.add(Ly.ReLU())
    m.add(Ly.Layer_Dense(12, 5))
    m.add(Ly.SoftMax())
    m.set(loss=Ly.Loss_CategoricalCrossEntropy(), optimizer=Ly.Optimizer_Adam(), accuracy=M.Accuracy_Categorical())
    m.finalize()
    m.load_parameters(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "checkpoint_cupy_format.pkl"))
    assert m.layers[9].weights.dtype == torch.float32       # float64 dense arrays are cast on load
    probs = m.predict(g["x"])
    assert O.rel_l2(host(probs), g["probs"]) <= 1e-5
    conv = m.layers[0]
    assert conv.weights is conv.filter_weights


def test_checkpoint_with_optimizer_state_resumes_training(env, tmp_path):
    torch, _lib, Ly, M = env
    rng = np.random.default_rng(17)
    a, shape = build(env, "fmnist", "bf16", True)
    batches = [(rng.random((8,) + shape).astype(np.float32), rng.integers(0, 10, 8)) for _ in range(3)]
    for X, y in batches[:2]:
        a.train_step(X, y)
    path = os.path.join(tmp_path, "ckpt")
    a.save_parameters(path, include_optimizer=True)
    b, _ = build(env, "fmnist", "bf16", True)
    b.load_parameters(path)
    assert b.optimizer.iterations == 2
    assert O.rel_l2(host(b.flat_m), host(a.flat_m)) <= 1e-7 and O.rel_l2(host(b.flat_v), host(a.flat_v)) <= 1e-7
    cache2 = host(a.layers[0].weight_cache).copy()
    a.train_step(*batches[2]); b.train_step(*batches[2])
    assert O.rel_l2(host(b.flat_params), host(a.flat_params)) <= 1e-6
    c, _ = build(env, "fmnist", "bf16", False)              # per-layer state (no flat buffers) resumes as well
    c.load_parameters(path)
    assert c.optimizer.iterations == 2 and O.rel_l2(host(c.layers[0].weight_cache), cache2) <= 1e-7


def test_block_tail_hands_operand_copies_to_neighbouring_layers(env):
    """finalize(fuse=True): the fused block tail (Batch_Norm + ReLU + pooling) writes the bf16 operand copy of its
    pooled output into the next layer's workspace (a Conv_Layer, or the Dense behind a Flatten) and, going back, the
    copy of its dx plus the bias-gradient column sums into the convolution in front -- those layers then run no cast
    pass.  Checked against the same model without the hand-off (identical tensor-core inputs, so the same numbers)
    and against the oracle's layer-by-layer chain."""
    torch, _lib, Ly, M = env

    def make(hand_off):
        np.random.seed(12)
        m = M.Model()
        m.add(Ly.Conv_Layer((16, 16, 16), 64, (3, 3), (1, 1), "same", math_mode="bf16"))
        m.add(Ly.Batch_Norm(n_features=64))
        m.add(Ly.ReLU())
        m.add(Ly.Pooling((2, 2), (2, 2), "valid", "max"))
        m.add(Ly.Conv_Layer((8, 8, 64), 96, (3, 3), (1, 1), "same", math_mode="bf16"))      # 96 channels: copy rows padded to 128
        m.add(Ly.Batch_Norm(n_features=96))
        m.add(Ly.Leaky_ReLU(0.1))
        m.add(Ly.Pooling((2, 2), (2, 2), "valid", "max"))
        m.add(Ly.Flatten())
        m.add(Ly.Layer_Dense(4 * 4 * 96, 32, math_mode="bf16"))
        m.add(Ly.Layer_Dense(32, 10, math_mode="bf16"))
        m.add(Ly.SoftMax())
        m.set(loss=Ly.Loss_CategoricalCrossEntropy(label_smoothing=0.01), optimizer=Ly.Optimizer_Adam(learning_rate=1e-3),
              accuracy=M.Accuracy_Categorical())
        m.finalize(flat=True, fuse=True)
        bns = [l for l in m.layers if isinstance(l, Ly.Batch_Norm)]
        assert isinstance(bns[0].copy_consumer, Ly.Conv_Layer) and isinstance(bns[1].copy_consumer, Ly.Layer_Dense)
        assert all(isinstance(b.copy_dy_consumer, Ly.Conv_Layer) for b in bns)
        if not hand_off:
            for b in bns:
                b.copy_consumer = b.copy_dy_consumer = None
        return m

    rng = np.random.default_rng(4)
    X = rng.standard_normal((6, 16, 16, 16)).astype(np.float32)
    y = rng.integers(0, 10, 6)
    with_copy, without = make(True), make(False)
    counts = []
    for m in (with_copy, without):
        m.forward(X, training=True)                      # sizes the workspaces
        n0 = _lib.launch_count()
        out = m.forward(X, training=True)
        m.backward(out, y)
        counts.append(_lib.launch_count() - n0)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    # two cast passes less going forward (conv 2, dense 1) and one less going back: the dy of conv 1; the tail behind
    # conv 2 has 96 channels, and the column sums that go with a dy copy need C/4 to divide 256, so conv 2 casts itself
    assert counts[1] - counts[0] == 3, counts
    assert O.rel_l2(host(with_copy.layers[-1].output), host(without.layers[-1].output)) <= 1e-6
    assert O.rel_l2(host(with_copy.flat_grads), host(without.flat_grads)) <= 1e-5
    conv2 = with_copy.layers[4]
    assert torch.equal(conv2.output, without.layers[4].output)      # the same bf16 operands went into the tensor cores
    # ... and both agree with the oracle's chain
    probs, grads = oracle_step(with_copy, Ly, X, y)
    assert O.rel_l2(host(with_copy.layers[-1].output), probs) <= 2e-2
    for k, (dw, db) in grads.items():                    # bf16 operands through six layers and two Batch_Norm backward passes: several per cent of the norm
        l = with_copy.layers[k]
        if not isinstance(l, Ly.Batch_Norm):
            assert O.rel_l2(host(l.dweights), dw) <= 1e-1, k
    # inference takes the same path (the copy is written by the evaluation pass too)
    e1 = with_copy.forward(X, training=False)
    e2 = without.forward(X, training=False)
    assert O.rel_l2(host(e1), host(e2)) <= 1e-6
    # an input the tail did not produce is cast by the layer itself
    other = torch.randn((6, 8, 8, 64), device="cuda")
    n0 = _lib.launch_count()
    conv2.forward(other, True)
    ref = Ly.Conv_Layer((8, 8, 64), 96, (3, 3), (1, 1), "same", math_mode="bf16")
    ref.set_parameters(conv2.filter_weights, conv2.biases)
    assert torch.equal(ref.forward(other, True), conv2.output)


def test_lean_mode_trains_to_the_same_parameters(env):
    """finalize(fuse=True, lean=True): fp32 tensors that only this library's next kernel would read -- and reads as a
    bf16 operand copy -- are not written.  The tensor cores get the same operands, so parameters, gradients and
    predictions are the same numbers; the skipped arrays are placeholders that a layer refuses to read."""
    torch, _lib, Ly, M = env
    rng = np.random.default_rng(6)

    def make(lean):
        np.random.seed(33)
        m = M.Model()
        c_in, hw = 16, 16
        for c_out in (64, 128):
            m.add(Ly.Conv_Layer((hw, hw, c_in), c_out, (3, 3), (1, 1), "same", math_mode="bf16"))
            m.add(Ly.Batch_Norm(n_features=c_out))
            m.add(Ly.ReLU())
            m.add(Ly.Pooling((2, 2), (2, 2), "valid", "max"))
            c_in, hw = c_out, hw // 2
        m.add(Ly.Flatten())
        m.add(Ly.Layer_Dense(4 * 4 * 128, 64, math_mode="bf16"))
        m.add(Ly.Layer_Dense(64, 10, math_mode="bf16"))
        m.add(Ly.SoftMax())
        m.set(loss=Ly.Loss_CategoricalCrossEntropy(label_smoothing=0.01), optimizer=Ly.Optimizer_Adam(learning_rate=1e-3),
              accuracy=M.Accuracy_Categorical())
        m.finalize(flat=True, fuse=True, lean=lean)
        return m

    lean, full = make(True), make(False)
    for _ in range(3):
        X = rng.standard_normal((8, 16, 16, 16)).astype(np.float32)
        y = rng.integers(0, 10, 8)
        lean.train_step(X, y)
        full.train_step(X, y)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert torch.equal(lean.flat_params, full.flat_params)
    assert torch.equal(lean.flat_grads, full.flat_grads)
    Xe = rng.standard_normal((8, 16, 16, 16)).astype(np.float32)
    assert torch.equal(lean.predict(Xe), full.predict(Xe))
    # the placeholders: the first tail's pooled output (x of conv 2) and the second tail's dx (dvalues of conv 2)
    bn1, bn2 = [l for l in lean.layers if isinstance(l, Ly.Batch_Norm)]
    assert getattr(bn1.output, "_aether_unwritten", False) and getattr(bn2.dinputs, "_aether_unwritten", False)
    foreign = Ly.Conv_Layer((8, 8, 64), 32, math_mode="bf16")
    with pytest.raises(_lib.AetherError):
        foreign.forward(bn1.output, True)                             # no copy of it in THAT layer's workspace


@pytest.mark.parametrize("lean", [False, True])
def test_first_layer_takes_the_dy_copy_from_its_block_tail(env, lean):
    """A first layer (3 input channels: thread-built operands) reads dvalues as the bf16 copy its block tail wrote,
    brought in by TMA already in operand form, and its bias gradient from the tail's column sums: same gradients as
    with the fp32 array converted inside the kernel."""
    torch, _lib, Ly, M = env

    def make(hand_off):
        np.random.seed(21)
        m = M.Model()
        m.add(Ly.Conv_Layer((16, 16, 3), 64, (3, 3), (1, 1), "same", math_mode="bf16"))
        m.add(Ly.Batch_Norm(n_features=64))
        m.add(Ly.ReLU())
        m.add(Ly.Pooling((2, 2), (2, 2), "valid", "max"))
        m.add(Ly.Flatten())
        m.add(Ly.Layer_Dense(8 * 8 * 64, 10, math_mode="bf16"))
        m.add(Ly.SoftMax())
        m.set(loss=Ly.Loss_CategoricalCrossEntropy(), optimizer=Ly.Optimizer_Adam(learning_rate=1e-3),
              accuracy=M.Accuracy_Categorical())
        m.finalize(flat=True, fuse=True, lean=lean and hand_off)
        bn = m.layers[1]
        assert bn.copy_dy_consumer is m.layers[0] and m.layers[0].first_in_model
        if not hand_off:
            bn.copy_dy_consumer = None
        return m

    rng = np.random.default_rng(2)
    X = rng.random((300, 16, 16, 3)).astype(np.float32)      # 600 tiles of 128 pixels: several per CTA, ragged last one
    y = rng.integers(0, 10, 300)
    a, b = make(True), make(False)
    for m in (a, b):
        out = m.forward(X, training=True)
        m.backward(out, y)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    ca, cb = a.layers[0], b.layers[0]
    assert O.rel_l2(host(ca.dweights), host(cb.dweights)) <= 1e-6
    assert np.abs(host(ca.dbiases) - host(cb.dbiases)).max() <= 1e-5 * np.abs(host(b.flat_grads)).max()   # ~0 in front of a Batch_Norm
    if lean:
        assert getattr(a.layers[1].dinputs, "_aether_unwritten", False)
    # asked for dinputs after all, the layer falls back to the fp32 array (which must exist then)
    if not lean:
        dx = ca.backward(a.layers[1].dinputs, need_dinputs=True)
        assert dx is not None and O.rel_l2(host(ca.dweights), host(cb.dweights)) <= 1e-6


@pytest.mark.parametrize("flat,fuse", [(False, False), (True, True)])
def test_whole_model_save_and_load(env, tmp_path, flat, fuse):
    """Model.save / Model.load (CNN_model_cupy.py:291-317): the loaded model predicts the same and goes on training
    to the same parameters as the one that was saved (Adam's moments and step count travel with it)."""
    torch, _lib, Ly, M = env
    rng = np.random.default_rng(40)
    m, shape = build(env, "cifar", "bf16", flat, fuse=fuse)
    m.enable_device_step() if flat else None
    batches = [(rng.random((8,) + shape).astype(np.float32), rng.integers(0, 10, 8)) for _ in range(3)]
    for X, y in batches[:2]:
        m.train_step(X, y)
    path = os.path.join(tmp_path, "whole_model")
    m.save(path)
    loaded = M.Model.load(path)
    assert [type(l).__name__ for l in loaded.layers] == [type(l).__name__ for l in m.layers]
    assert loaded.optimizer.iterations == 2 and (loaded.flat_params is not None) == flat
    assert not hasattr(loaded.layers[0], "output") or loaded.layers[0].__dict__.get("output") is None
    Xe = rng.random((8,) + shape).astype(np.float32)
    assert O.rel_l2(host(loaded.predict(Xe)), host(m.predict(Xe))) <= 1e-6
    if flat:
        loaded.enable_device_step()
        for a, b in zip(m.layers, loaded.layers):          # the same dropout streams from here on
            if hasattr(a, "seed"):
                assert a.seed == b.seed
        m.train_step(*batches[2]); loaded.train_step(*batches[2])
        assert O.rel_l2(host(loaded.flat_params), host(m.flat_params)) <= 1e-6
        assert O.rel_l2(host(loaded.flat_m), host(m.flat_m)) <= 1e-6
