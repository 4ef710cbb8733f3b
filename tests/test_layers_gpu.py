"""GPU parity tests of the bandwidth-bound layers, Dense, softmax/loss and Adam (through the C ABI)
against the golden vectors of the reference's classes and the NumPy oracle."""
import numpy as np
import pytest

from oracle import aether_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    import torch
    from aether_ml_b200 import _lib, layers
    if not torch.cuda.is_available():
        pytest.fail("CUDA device required for -m gpu tests")
    return torch, _lib, layers


def host(t):
    return t.detach().cpu().numpy()


@pytest.mark.parametrize("name", ["bn_4d", "bn_2d"])
def test_batch_norm_golden(env, golden, name):
    torch, _lib, layers = env
    g = golden(name)
    bn = layers.Batch_Norm(epsilon=1e-5, momentum=0.9)
    bn.forward(g["x"], True)                               # first call creates gamma/beta/running stats
    assert O.rel_l2(host(bn.output), g["y_first"]) <= 1e-5
    bn.gamma.copy_(torch.from_numpy(g["gamma"])); bn.beta.copy_(torch.from_numpy(g["beta"]))
    y = bn.forward(g["x"], True)
    assert O.rel_l2(host(y), g["y"]) <= 1e-5
    assert O.rel_l2(host(bn.batch_mean), g["mean"]) <= 1e-5 and O.rel_l2(host(bn.batch_var), g["var"]) <= 1e-5
    assert host(bn.running_mean).shape == g["rm1"].shape
    assert O.rel_l2(host(bn.running_mean), g["rm1"]) <= 1e-5 and O.rel_l2(host(bn.running_var), g["rv1"]) <= 1e-5
    dx = bn.backward(g["dy"])
    assert O.rel_l2(host(dx), g["dx"]) <= 1e-4
    assert O.rel_l2(host(bn.dweights), g["dgamma"]) <= 1e-5 and O.rel_l2(host(bn.dbiases), g["dbeta"]) <= 1e-5
    ye = bn.forward(g["x"], False)
    assert O.rel_l2(host(ye), g["y_eval"]) <= 1e-5
    assert bn.weights is bn.gamma and bn.biases is bn.beta
    params = bn.get_parameters()
    bn2 = layers.Batch_Norm()
    bn2.set_parameters(*params)
    assert O.rel_l2(host(bn2.forward(g["x"], False)), g["y_eval"]) <= 1e-5


@pytest.mark.parametrize("shape", [(128, 32, 32, 32), (64, 7, 7, 64), (37, 5, 3, 10), (512, 256), (3, 2, 2, 300)])
def test_batch_norm_shapes(env, shape):
    torch, _lib, layers = env
    rng = np.random.default_rng(2)
    x = (rng.standard_normal(shape) * 3 + 10).astype(np.float32)      # large mean: exercises the shifted sums
    dy = rng.standard_normal(shape).astype(np.float32)
    C = shape[-1]
    gamma = (rng.standard_normal(C) + 1).astype(np.float32); beta = rng.standard_normal(C).astype(np.float32)
    bn = layers.Batch_Norm(n_features=C)
    bn.gamma.copy_(torch.from_numpy(gamma)); bn.beta.copy_(torch.from_numpy(beta))
    y = bn.forward(x, True)
    yo, _, mean, var, rm, rv = O.bn_forward_train(x, gamma, beta, np.zeros(C), np.ones(C))
    assert O.rel_l2(host(y), yo) <= 2e-5
    assert O.rel_l2(host(bn.batch_var), var) <= 1e-4
    assert O.rel_l2(host(bn.running_var), rv) <= 1e-5
    dx = bn.backward(dy)
    dxo, dgo, dbo = O.bn_backward(x, dy, gamma, mean, var)
    assert O.rel_l2(host(dx), dxo) <= 2e-4
    assert O.rel_l2(host(bn.dweights), dgo) <= 1e-4 and O.rel_l2(host(bn.dbiases), dbo) <= 1e-4


# (S, H, W, Cin, Cout, mode, statistics expected from the conv epilogue)
@pytest.mark.parametrize("case", [(8, 32, 32, 64, 128, "bf16", True), (37, 20, 24, 64, 64, "tf32", True),
                                  (300, 32, 32, 3, 64, "bf16", True), (5, 28, 28, 1, 32, "bf16", True),
                                  (200, 32, 32, 3, 128, "bf16", True), (6, 20, 20, 3, 256, "bf16", True),
                                  (3, 16, 16, 2, 192, "bf16", True),
                                  # per-tap tensor-core kernel: one / two / three column tiles, ragged pixel tiles
                                  (16, 8, 8, 256, 256, "bf16", True), (40, 8, 8, 128, 512, "bf16", True),
                                  (50, 16, 16, 128, 256, "bf16", True), (7, 10, 10, 32, 96, "tf32", True),
                                  (3, 5, 7, 32, 40, "bf16", True), (700, 6, 6, 16, 96, "bf16", True),
                                  # per-tap kernel on CTA pairs: odd number of pixel tiles, two column tiles, TF32
                                  (61, 24, 24, 128, 256, "bf16", True), (300, 8, 8, 128, 512, "bf16", True),
                                  (149, 16, 16, 64, 256, "tf32", True),
                                  # window kernel on CTA pairs (TF32 filter too large for one CTA; odd number of strips)
                                  (11, 54, 56, 64, 128, "tf32", True),
                                  (4, 12, 12, 8, 16, "fp32", False)])
def test_batch_norm_statistics_from_conv_epilogue(env, case):
    """Conv_Layer -> Batch_Norm with the batch statistics taken in the convolution's epilogue: same result as
    Batch_Norm's own reduction over the layer output (CNN_classes_cupy.py:467-476), bias far from zero included."""
    torch, _lib, layers = env
    S, H, W, Cin, Cout, mode, expect = case
    rng = np.random.default_rng(5)
    np.random.seed(5)
    x = rng.standard_normal((S, H, W, Cin)).astype(np.float32)
    conv = layers.Conv_Layer((H, W, Cin), Cout, (3, 3), (1, 1), "same", math_mode=mode)
    conv.biases.copy_(torch.from_numpy((rng.standard_normal(Cout) * 4 + 3).astype(np.float32)))
    gamma = (rng.standard_normal(Cout) + 1).astype(np.float32); beta = rng.standard_normal(Cout).astype(np.float32)
    bn = layers.Batch_Norm(n_features=Cout)
    bn.gamma.copy_(torch.from_numpy(gamma)); bn.beta.copy_(torch.from_numpy(beta))
    conv.emit_bn_stats = True
    bn.stats_from = conv
    y = conv.forward(x, True)
    assert (conv.bn_partials is not None) == expect
    z = bn.forward(y, True)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    zo, _, mean, var, rm, rv = O.bn_forward_train(host(y), gamma, beta, np.zeros(Cout), np.ones(Cout))
    assert O.rel_l2(host(bn.batch_mean), mean) <= 1e-5
    assert O.rel_l2(host(bn.batch_var), var) <= 1e-4
    assert O.rel_l2(host(bn.running_mean), rm) <= 1e-5 and O.rel_l2(host(bn.running_var), rv) <= 1e-4
    assert O.rel_l2(host(z), zo) <= 5e-5
    # a Batch_Norm fed something else than that convolution's output must ignore the partials
    other = (rng.standard_normal(tuple(y.shape)) * 2 - 1).astype(np.float32)
    z2 = bn.forward(other, True)
    zo2 = O.bn_forward_train(other, gamma, beta, np.zeros(Cout), np.ones(Cout))[0]
    assert O.rel_l2(host(z2), zo2) <= 2e-5
    # inference keeps using the running statistics
    conv.forward(x, False)
    assert conv.bn_partials is None


# inputs whose convolution outputs have |mean| >> std per channel: a large offset, raw 0..255 pixels, |N(0,1)|
@pytest.mark.parametrize("kind", ["offset50", "pixels", "abs"])
@pytest.mark.parametrize("case", [(8, 32, 32, 64, 128, "bf16"),        # halo kernel
                                  (50, 16, 16, 128, 256, "bf16"),      # per-tap kernel
                                  (37, 20, 24, 64, 64, "tf32"),        # halo kernel, TF32
                                  (200, 32, 32, 3, 128, "bf16"),       # first layer on the tensor cores
                                  (64, 28, 28, 1, 32, "fp32")])        # first layer on the CUDA cores
def test_conv_epilogue_statistics_with_nonzero_mean_outputs(env, case, kind):
    """The epilogue statistics sum about a per-column pivot (the mean of the first tile), so a channel whose mean is
    far from zero compared with its spread keeps its variance: same 1e-4 tolerance as for centred data, against the
    oracle's Batch_Norm statistics of the very tensor the convolution wrote."""
    torch, _lib, layers = env
    S, H, W, Cin, Cout, mode = case
    rng = np.random.default_rng(9)
    np.random.seed(9)
    base = rng.standard_normal((S, H, W, Cin))
    x = {"offset50": base + 50.0, "pixels": np.floor(rng.random((S, H, W, Cin)) * 256.0), "abs": np.abs(base)}[kind]
    x = x.astype(np.float32)
    conv = layers.Conv_Layer((H, W, Cin), Cout, (3, 3), (1, 1), "same", math_mode=mode)
    # all-positive filters push every channel's mean far from zero (a zero-mean filter would cancel the offset)
    conv.filter_weights.copy_(conv.filter_weights.abs())
    bn = layers.Batch_Norm(n_features=Cout)
    conv.emit_bn_stats = True
    bn.stats_from = conv
    y = conv.forward(x, True)
    assert conv.bn_partials is not None
    bn.forward(y, True)
    torch.cuda.synchronize()
    yh = host(y).astype(np.float64).reshape(-1, Cout)
    mean, var = yh.mean(axis=0), yh.var(axis=0)
    assert np.median(np.abs(mean) / np.sqrt(var)) > 3.0          # the case is what it claims to be
    assert O.rel_l2(host(bn.batch_mean), mean) <= 1e-5
    assert O.rel_l2(host(bn.batch_var), var) <= 1e-4


@pytest.mark.parametrize("case", [(6, 8, 12, 32, 0.0, (2, 2), True), (3, 12, 6, 64, 0.01, (2, 2), False),
                                  (2, 9, 6, 8, 0.2, (3, 3), True)])
def test_fused_block_tail_matches_oracle_chain(env, case):
    """Batch_Norm + (Leaky_)ReLU + spatial dropout + tiling max pooling in one pass each way (block_fused.cu) against
    the oracle's layer-by-layer chain: pooled output, argmax, dX, dgamma, dbeta; inference path too."""
    torch, _lib, layers = env
    S, H, W, C, alpha, f, with_drop = case
    rng = np.random.default_rng(13)
    x = (rng.standard_normal((S, H, W, C)) * 2 + 0.5).astype(np.float32)
    gamma = (rng.standard_normal(C) + 1).astype(np.float32); beta = rng.standard_normal(C).astype(np.float32)
    mask = ((rng.random(C) < 0.7) / 0.7).astype(np.float32)            # some channels dropped, the rest scaled up
    bn = layers.Batch_Norm(n_features=C)
    bn.gamma.copy_(torch.from_numpy(gamma)); bn.beta.copy_(torch.from_numpy(beta))
    act = layers.Leaky_ReLU(alpha) if alpha else layers.ReLU()
    drop = layers.Layer_Dropout_Spatial(0.3)
    drop.fixed_mask = mask
    pool = layers.Pooling(f, f, "valid", "max")
    bn.fused_alpha = float(alpha); act.fused_into_prev = True
    if with_drop:
        bn.fused_dropout = drop; drop.fused_into_prev = True
    bn.fused_pool = pool; pool.fused_bn = bn
    chain = [bn, act] + ([drop] if with_drop else []) + [pool]
    out = x
    for l in chain:
        out = l.forward(out, True)
    assert bn.pooled_now and tuple(out.shape) == (S, H // f[0], W // f[1], C)
    # oracle: the same four layers one after the other
    yb, _, mean, var, rm, rv = O.bn_forward_train(x, gamma, beta, np.zeros(C), np.ones(C))
    ya = O.leaky_relu_forward(yb, alpha) if alpha else O.relu_forward(yb)
    yd = ya * mask if with_drop else ya
    yp, arg = O.pool_forward(yd, f, f)
    assert O.rel_l2(host(out), yp) <= 1e-5
    assert O.rel_l2(host(bn.running_mean), rm) <= 1e-5 and O.rel_l2(host(bn.running_var), rv) <= 1e-4
    dyp = rng.standard_normal(yp.shape).astype(np.float32)
    g = dyp
    for l in reversed(chain):
        g = l.backward(g)
    torch.cuda.synchronize()
    gd = O.pool_backward(dyp, yd.shape, arg, f, f)
    if with_drop:
        gd = gd * mask
    ga = O.leaky_relu_backward(yb, gd, alpha) if alpha else O.relu_backward(yb, gd)
    dxo, dgo, dbo = O.bn_backward(x, ga, gamma, mean, var)
    assert O.rel_l2(host(g), dxo) <= 2e-4
    assert O.rel_l2(host(bn.dweights), dgo) <= 1e-4 and O.rel_l2(host(bn.dbiases), dbo) <= 1e-4
    # inference: running statistics, no mask
    oe = x
    for l in chain:
        oe = l.forward(oe, False)
    ye = O.bn_forward_eval(x, gamma, beta, host(bn.running_mean), host(bn.running_var))
    ye = O.leaky_relu_forward(ye, alpha) if alpha else O.relu_forward(ye)
    assert O.rel_l2(host(oe), O.pool_forward(ye, f, f)[0]) <= 1e-5


@pytest.mark.parametrize("alpha", [0.0, 0.1])
def test_fused_activation_gradient_at_zero_preactivation(env, alpha):
    """Batch_Norm + (Leaky_)ReLU in the same passes, no pooling: where the pre-activation is exactly 0 the reference
    lets the gradient through (ReLU.backward zeroes only inputs < 0, CNN_classes_cupy.py:412-414).  Channel 0 is
    constant with beta = 0, so every one of its pre-activations is exactly 0; the other channels are ordinary."""
    torch, _lib, layers = env
    S, H, W, C = 4, 6, 5, 8
    rng = np.random.default_rng(21)
    x = rng.standard_normal((S, H, W, C)).astype(np.float32)
    x[..., 0] = 1.5
    gamma = (rng.random(C) + 0.5).astype(np.float32); beta = rng.standard_normal(C).astype(np.float32)
    beta[0] = 0.0
    bn = layers.Batch_Norm(n_features=C)
    bn.gamma.copy_(torch.from_numpy(gamma)); bn.beta.copy_(torch.from_numpy(beta))
    bn.fused_alpha = float(alpha)
    y = bn.forward(x, True)
    yb, _, mean, var, _, _ = O.bn_forward_train(x, gamma, beta, np.zeros(C), np.ones(C))
    assert np.all(yb[..., 0] == 0.0)
    ya = O.leaky_relu_forward(yb, alpha) if alpha else O.relu_forward(yb)
    assert O.rel_l2(host(y), ya) <= 1e-5
    dy = rng.standard_normal(x.shape).astype(np.float32)
    dx = bn.backward(dy)
    ga = O.leaky_relu_backward(yb, dy, alpha) if alpha else O.relu_backward(yb, dy)
    assert np.array_equal(ga[..., 0], dy[..., 0])                       # the oracle passes the gradient at 0
    dxo, dgo, dbo = O.bn_backward(x, ga, gamma, mean, var)
    assert O.rel_l2(host(bn.dbiases), dbo) <= 1e-5                      # dbeta[0] = sum(dy[..., 0]): not blocked
    assert abs(float(bn.dbiases[0]) - float(dy[..., 0].sum())) <= 1e-4 * np.abs(dy[..., 0]).sum()
    assert O.rel_l2(host(bn.dweights)[1:], dgo[1:]) <= 1e-4
    assert O.rel_l2(host(dx)[..., 1:], dxo[..., 1:]) <= 2e-4


@pytest.mark.parametrize("name", ["pool_max_2x2", "pool_max_odd", "pool_max_overlap", "pool_avg_2x2"])
def test_pooling_golden(env, golden, name):
    torch, _lib, layers = env
    g = golden(name)
    f = tuple(int(v) for v in g["filter_size"]); st = tuple(int(v) for v in g["strides"]); kind = str(g["kind"])
    pool = layers.Pooling(f, st, "valid", kind)
    y = pool.forward(g["x"], True)
    if kind == "max":
        assert np.array_equal(host(y), g["y"])                         # bit exact
        rows, cols = pool.max_indicies
        assert np.array_equal(host(rows), g["arg_rows"]) and np.array_equal(host(cols), g["arg_cols"])
    else:
        assert O.rel_l2(host(y), g["y"]) <= 1e-6
    dx = pool.backward(g["dy"])
    assert dx.shape == g["x"].shape
    assert O.rel_l2(host(dx), g["dx"]) <= 1e-6


def test_pooling_notebook_example_and_shapes(env):
    torch, _lib, layers = env
    x = np.array([[1, 2, 3, 4], [4, 5, 6, 5], [7, 8, 9, 6], [8, 7, 6, 5]], np.float32)[None, :, :, None]
    pool = layers.Pooling()
    assert np.array_equal(host(pool.forward(x, True))[0, :, :, 0], [[5, 6], [8, 9]])
    avg = layers.Pooling(pooling_type="average")
    assert np.array_equal(host(avg.forward(x, True))[0, :, :, 0], [[3, 4.5], [7.5, 6.5]])
    rng = np.random.default_rng(0)
    for shape in [(128, 32, 32, 32), (16, 7, 7, 64), (3, 9, 11, 5)]:
        xx = np.maximum(rng.standard_normal(shape), 0).astype(np.float32)    # post-ReLU: many all-zero windows
        p = layers.Pooling()
        y = p.forward(xx, True)
        yo, arg = O.pool_forward(xx)
        assert np.array_equal(host(y), yo.astype(np.float32))
        dy = rng.standard_normal(yo.shape).astype(np.float32)
        assert np.array_equal(host(p.backward(dy)), O.pool_backward(dy, shape, arg).astype(np.float32))
    with pytest.raises(ValueError):
        layers.Pooling().forward(np.zeros((4, 4, 4), np.float32), True)
    with pytest.raises(ValueError):
        layers.Pooling(padding="same").forward(np.zeros((1, 4, 4, 4), np.float32), True)


def test_elementwise_golden(env, golden):
    torch, _lib, layers = env
    g = golden("elementwise")
    relu = layers.ReLU()
    assert np.array_equal(host(relu.forward(g["x"], True)), g["relu_y"])
    assert np.array_equal(host(relu.backward(g["dy"])), g["relu_dx"])
    lr = layers.Leaky_ReLU(0.01)
    assert O.rel_l2(host(lr.forward(g["x"], True)), g["lrelu_y"]) <= 1e-6
    assert O.rel_l2(host(lr.backward(g["dy"])), g["lrelu_dx"]) <= 1e-6
    sd = layers.Layer_Dropout_Spatial(float(g["sd_rate"]))
    sd.fixed_mask = g["sd_mask"]
    assert O.rel_l2(host(sd.forward(g["x"], True)), g["sd_y"]) <= 1e-6
    assert O.rel_l2(host(sd.backward(g["dy"])), g["sd_dx"]) <= 1e-6
    assert np.array_equal(host(sd.forward(g["x"], False)), g["x"])
    # odd sizes: vector body + scalar tail
    x = np.random.default_rng(1).standard_normal(1003).astype(np.float32)
    assert np.array_equal(host(layers.ReLU().forward(x, True)), np.maximum(x, 0))


def test_dropout_statistics(env):
    torch, _lib, layers = env
    d = layers.Layer_Dropout(0.25, seed=9)
    x = np.ones((512, 1024), np.float32)
    y = host(d.forward(x, True))
    keep = 0.75
    assert set(np.unique(y)).issubset({0.0, np.float32(1 / keep)})
    assert abs((y > 0).mean() - keep) < 5e-3
    y2 = host(d.forward(x, True))
    assert not np.array_equal(y, y2)                                   # a new mask every call
    dy = np.full_like(x, 2.0)
    assert np.array_equal(host(d.backward(dy)), y2 * 2.0)
    assert np.array_equal(host(d.forward(x, False)), x)
    spatial = layers.Layer_Dropout_Spatial(0.5)
    ys = host(spatial.forward(np.ones((4, 3, 3, 64), np.float32), True))
    assert np.all(ys == ys[0, 0, 0])                                   # one decision per channel for the whole batch


@pytest.mark.parametrize("mode,tol", [("fp32", 1e-5), ("tf32", 1e-3), ("bf16", 1e-2)])
def test_dense_softmax_loss_adam_golden(env, golden, mode, tol):
    torch, _lib, layers = env
    g = golden("dense_loss_adam")
    dense = layers.Layer_Dense(12, 10, weight_regularizer_l2=2e-5, bias_regularizer_l2=1e-5, math_mode=mode)
    dense.set_parameters(g["w0"], g["b0"])
    z = dense.forward(g["x"], True)
    assert O.rel_l2(host(z), g["z"]) <= 1e-5                             # 12 -> 10 always takes the fp32 kernel
    sm = layers.SoftMax()
    p = sm.forward(z, True)
    assert O.rel_l2(host(p), g["p"]) <= 1e-5
    loss = layers.Loss_CategoricalCrossEntropy(0.01)
    assert O.rel_l2(host(loss.forward(p, g["labels"], True)), g["sample_losses"]) <= 1e-5
    comb = layers.Activation_Softmax_Loss_CategoricalCrossEntropy(0.01)
    dz = comb.backward(p, g["labels"], training=True)
    assert O.rel_l2(host(dz), g["dz"]) <= 1e-5
    onehot = np.eye(10, dtype=np.float32)[g["labels"]]
    assert np.array_equal(host(comb.backward(p, onehot, training=True)), host(dz))
    dense.backward(dz)
    assert O.rel_l2(host(dense.dinputs), g["dx"]) <= 1e-5
    assert O.rel_l2(host(dense.dweights), g["dw"]) <= 1e-5 and O.rel_l2(host(dense.dbiases), g["db"]) <= 1e-5
    assert (sm.predictions(p).cpu().numpy() == g["p"].argmax(1)).all()
    opt = layers.Optimizer_Adam(learning_rate=1e-3, decay=5e-5)
    for it in range(3):
        opt.pre_update_parameters()
        opt.update_parameters(dense)
        opt.post_update_parameters()
        assert np.isclose(opt.current_learning_rate, g["lrs"][it])
        assert O.rel_l2(host(dense.weights), g["w_hist"][it]) <= 1e-6
        assert O.rel_l2(host(dense.biases), g["b_hist"][it]) <= 2e-5      # fp32 state vs the reference's fp64
    assert O.rel_l2(host(dense.weight_momentums), g["m_w"]) <= 1e-5 and O.rel_l2(host(dense.weight_cache), g["v_w"]) <= 5e-5


@pytest.mark.parametrize("mode,tol", [("tf32", 1e-3), ("bf16", 1e-2)])
def test_dense_tensor_core(env, mode, tol):
    torch, _lib, layers = env
    rng = np.random.default_rng(8)
    np.random.seed(8)
    dense = layers.Layer_Dense(2048, 256, math_mode=mode)
    w = (rng.standard_normal((2048, 256)) * 0.03).astype(np.float32); b = rng.standard_normal((1, 256)).astype(np.float32)
    dense.set_parameters(w, b)
    x = rng.standard_normal((128, 2048)).astype(np.float32); dy = rng.standard_normal((128, 256)).astype(np.float32)
    y = dense.forward(x, True); dense.backward(dy)
    dxo, dwo, dbo = O.dense_backward(x, w, b, dy)
    assert O.rel_l2(host(y), O.dense_forward(x, w, b)) <= tol
    assert O.rel_l2(host(dense.dinputs), dxo) <= tol and O.rel_l2(host(dense.dweights), dwo) <= tol
    assert O.rel_l2(host(dense.dbiases), dbo) <= 1e-5 and dense.dbiases.shape == (1, 256)


@pytest.mark.parametrize("shape", [(512, 1024, 10), (37, 132, 7), (5, 256, 12), (64, 8192, 3)])
def test_dense_classifier_head(env, shape):
    """Dense layers with very few outputs (the 10-class head of the reference's networks) run a warp-per-row forward
    on the CUDA cores in every math mode: fp32 results against the oracle."""
    torch, _lib, layers = env
    rows, n_in, n_out = shape
    rng = np.random.default_rng(rows)
    x = rng.standard_normal((rows, n_in)).astype(np.float32)
    dy = rng.standard_normal((rows, n_out)).astype(np.float32)
    np.random.seed(1)
    dense = layers.Layer_Dense(n_in, n_out, math_mode="bf16")
    dense.weights.copy_(torch.from_numpy(rng.standard_normal((n_in, n_out)).astype(np.float32) * 0.1))
    dense.biases.copy_(torch.from_numpy(rng.standard_normal((1, n_out)).astype(np.float32)))
    w, b = host(dense.weights), host(dense.biases)
    y = dense.forward(x, True)
    dx = dense.backward(dy)
    assert O.rel_l2(host(y), O.dense_forward(x, w, b)) <= 1e-5
    dxo, dwo, dbo = O.dense_backward(x, w, b, dy)
    assert O.rel_l2(host(dx), dxo) <= 1e-5 and O.rel_l2(host(dense.dweights), dwo) <= 1e-5
    assert O.rel_l2(host(dense.dbiases), dbo) <= 1e-5


def test_regularization_loss(env):
    torch, _lib, layers = env
    np.random.seed(1)
    d1 = layers.Layer_Dense(64, 32, weight_regularizer_l2=2e-5, bias_regularizer_l1=1e-3)
    d1.biases.copy_(torch.randn(1, 32))
    loss = layers.Loss_CategoricalCrossEntropy()
    loss.remember_trainable_layers([d1])
    w = host(d1.weights).astype(np.float64); b = host(d1.biases).astype(np.float64)
    expect = 2e-5 * (w * w).sum() + 1e-3 * np.abs(b).sum()
    assert np.isclose(float(loss.regularization_loss()), expect, rtol=1e-5)


def test_softmax_standalone_backward(env, golden):
    """SoftMax.backward on its own (the reference's per-sample Jacobian loop, CNN_classes_cupy.py:549-560)."""
    torch, _lib, layers = env
    g = golden("softmax_backward")
    sm = layers.SoftMax()
    p = sm.forward(g["z"].astype(np.float32), True)
    assert O.rel_l2(host(p), g["p"]) <= 1e-6
    dx = sm.backward(g["dvalues"].astype(np.float32))
    assert O.rel_l2(host(dx), g["dinputs"]) <= 1e-5
    rng = np.random.default_rng(3)
    z = rng.standard_normal((300, 1000)).astype(np.float32) * 3
    dv = rng.standard_normal((300, 1000)).astype(np.float32)
    p = sm.forward(z, True)
    assert O.rel_l2(host(sm.backward(dv)), O.softmax_backward(host(p), dv)) <= 1e-5
    with pytest.raises(ValueError):
        sm.backward(dv[:, :10])


def test_cross_entropy_with_rows_of_target_probabilities(env):
    """2-D targets -- one-hot rows and soft rows -- are used as they are by the loss and its gradients
    (CNN_classes_cupy.py:625-637, 644-650, 672-680), label smoothing applied on top."""
    torch, _lib, layers = env
    rng = np.random.default_rng(12)
    z = rng.standard_normal((33, 10)).astype(np.float32) * 2
    p = O.softmax(z)
    idx = rng.integers(0, 10, 33)
    onehot = np.eye(10)[idx]
    soft = rng.random((33, 10)); soft /= soft.sum(axis=1, keepdims=True)
    for smooth in (0.0, 0.05):
        loss = layers.Loss_CategoricalCrossEntropy(label_smoothing=smooth)
        comb = layers.Activation_Softmax_Loss_CategoricalCrossEntropy(label_smoothing=smooth)
        for tgt in (onehot, soft):
            got = loss.forward(p.astype(np.float32), tgt.astype(np.float32), training=True)
            assert O.rel_l2(host(got), O.cce_loss(p, tgt, smooth)) <= 1e-5
            dz = comb.backward(p.astype(np.float32), tgt.astype(np.float32))
            assert O.rel_l2(host(dz), O.softmax_cce_backward(p, tgt, smooth)) <= 1e-5
        # one-hot rows and class indices are the same targets
        a = comb.backward(p.astype(np.float32), onehot.astype(np.float32)).clone()
        b = comb.backward(p.astype(np.float32), idx)
        assert torch.equal(a, b)
