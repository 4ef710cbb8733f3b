"""CPU tests: the NumPy oracle against the golden vectors produced by the reference's own
NumPy classes and against the notebook known answers."""
import numpy as np
import pytest

from oracle import aether_oracle as O

CONV_CASES = ["conv_same_3x3", "conv_valid_3x3", "conv_same_5x5", "conv_stride2_valid",
              "conv_tensor_path_small", "conv_cfg1_tiny"]


@pytest.mark.parametrize("name", CONV_CASES)
def test_conv_matches_reference_vectors(golden, name):
    g = golden(name)
    st = tuple(int(v) for v in g["strides"]); pad = str(g["padding"])
    y = O.conv_forward(g["x"], g["w"], g["b"], st, pad)
    dx, dw, db = O.conv_backward(g["x"], g["w"], g["dy"], st, pad)
    assert y.shape == g["y"].shape
    assert O.rel_l2(y, g["y"]) < 1e-6
    assert O.rel_l2(dw, g["dw"]) < 1e-6
    assert O.rel_l2(db, g["db"]) < 1e-6
    assert O.rel_l2(dx, g["dx"]) < 1e-6
    # tap-by-tap BLAS evaluation is the same function
    yb = O.conv_forward_blas(g["x"], g["w"], g["b"], st, pad, dtype=np.float64)
    dxb, dwb, dbb = O.conv_backward_blas(g["x"], g["w"], g["dy"], st, pad, dtype=np.float64)
    for a, b in ((yb, y), (dxb, dx), (dwb, dw), (dbb, db)):
        assert O.rel_l2(a, b) < 1e-10


@pytest.mark.parametrize("name", ["conv_same_3x3", "conv_valid_3x3", "conv_stride2_valid"])
def test_conv_reference_numpy_dinputs_is_last_writer(golden, name):
    """The verbatim NumPy dinputs is NOT the scatter-add; it equals the last-writer model."""
    g = golden(name)
    st = tuple(int(v) for v in g["strides"]); pad = str(g["padding"])
    lw = O.conv_dinputs_last_writer(g["x"], g["w"], g["dy"], st, pad)
    assert O.rel_l2(lw, g["dx_verbatim"]) < 1e-6
    if name != "conv_stride2_valid":
        assert O.rel_l2(g["dx"], g["dx_verbatim"]) > 0.3


def test_conv_adjoint_identities():
    rng = np.random.default_rng(5)
    x = rng.standard_normal((2, 6, 7, 3)); w = rng.standard_normal((3, 3, 3, 4)); dy = rng.standard_normal((2, 6, 7, 4))
    y = O.conv_forward(x, w, np.zeros(4))
    dx, dw, db = O.conv_backward(x, w, dy)
    assert np.isclose((y * dy).sum(), (x * dx).sum(), rtol=1e-10)
    assert np.isclose((y * dy).sum(), (w * dw).sum(), rtol=1e-10)


def test_conv_finite_difference():
    rng = np.random.default_rng(6)
    x = rng.standard_normal((1, 4, 4, 2)); w = rng.standard_normal((3, 3, 2, 2)); dy = rng.standard_normal((1, 4, 4, 2))
    dx, dw, _ = O.conv_backward(x, w, dy)
    eps = 1e-6
    for idx in [(0, 0, 0, 0), (0, 2, 3, 1), (0, 3, 3, 0)]:
        xp = x.copy(); xp[idx] += eps; xm = x.copy(); xm[idx] -= eps
        fd = ((O.conv_forward(xp, w, np.zeros(2)) - O.conv_forward(xm, w, np.zeros(2))) * dy).sum() / (2 * eps)
        assert np.isclose(fd, dx[idx], rtol=1e-6)


def test_notebook_known_answers(golden):
    g = golden("notebook_kat")
    y = O.conv_forward(g["image"][None, :, :, None], g["kernel"][:, :, None, None], np.zeros(1))
    assert np.array_equal(y[0, :, :, 0], g["expected"])
    ones = np.ones((1, 5, 5, 1))
    assert np.all(O.conv_forward(ones, np.ones((3, 3, 1, 1)), [0.0], padding="valid") == 9)
    assert O.conv_forward(ones, np.ones((3, 3, 1, 1)), [0.0], padding="valid").shape == (1, 3, 3, 1)
    assert np.all(O.conv_forward(np.ones((1, 5, 5, 3)), np.ones((3, 3, 3, 1)), [0.0], padding="valid") == 27)
    w2 = np.ones((3, 3, 1, 2)); w2[..., 1] = 2
    y2 = O.conv_forward(ones, w2, [0.0, 0.0], padding="valid")
    assert np.all(y2[..., 0] == 9) and np.all(y2[..., 1] == 18)


def test_notebook_pooling_examples():
    x = np.array([[1, 2, 3, 4], [4, 5, 6, 5], [7, 8, 9, 6], [8, 7, 6, 5]], dtype=np.float64)[None, :, :, None]
    y, arg = O.pool_forward(x)
    assert np.array_equal(y[0, :, :, 0], [[5, 6], [8, 9]])
    ya, _ = O.pool_forward(x, pooling_type="average")
    assert np.array_equal(ya[0, :, :, 0], [[3, 4.5], [7.5, 6.5]])
    dxa = O.pool_backward(ya, x.shape, None, pooling_type="average")
    assert np.allclose(dxa[0, :2, :2, 0], 0.75) and np.allclose(dxa[0, :2, 2:, 0], 1.125)
    assert np.allclose(dxa[0, 2:, :2, 0], 1.875) and np.allclose(dxa[0, 2:, 2:, 0], 1.625)


@pytest.mark.parametrize("name", ["bn_4d", "bn_2d"])
def test_batch_norm(golden, name):
    g = golden(name)
    y, xhat, mean, var, rm, rv = O.bn_forward_train(g["x"], g["gamma"], g["beta"], g["rm0"], g["rv0"])
    assert O.rel_l2(y, g["y"]) < 1e-6 and O.rel_l2(mean, g["mean"]) < 1e-6 and O.rel_l2(var, g["var"]) < 1e-6
    assert O.rel_l2(rm, g["rm1"]) < 1e-6 and O.rel_l2(rv, g["rv1"]) < 1e-6
    dx, dg, dbeta = O.bn_backward(g["x"], g["dy"], g["gamma"], mean, var)
    assert O.rel_l2(dx, g["dx"]) < 1e-5 and O.rel_l2(dg, g["dgamma"]) < 1e-6 and O.rel_l2(dbeta, g["dbeta"]) < 1e-6
    ye = O.bn_forward_eval(g["x"], g["gamma"], g["beta"], g["rm1"], g["rv1"])
    assert O.rel_l2(ye, g["y_eval"]) < 1e-6


@pytest.mark.parametrize("name", ["pool_max_2x2", "pool_max_odd", "pool_max_overlap", "pool_avg_2x2"])
def test_pooling(golden, name):
    g = golden(name)
    f = tuple(int(v) for v in g["filter_size"]); st = tuple(int(v) for v in g["strides"]); kind = str(g["kind"])
    y, arg = O.pool_forward(g["x"], f, st, kind)
    if kind == "max":
        assert np.array_equal(y.astype(np.float32), g["y"])
    else:
        assert O.rel_l2(y, g["y"]) < 1e-6
    if kind == "max":
        assert np.array_equal(arg[0], g["arg_rows"]) and np.array_equal(arg[1], g["arg_cols"])
    dx = O.pool_backward(g["dy"], g["x"].shape, arg, f, st, kind)
    assert O.rel_l2(dx, g["dx"]) < 1e-6


def test_elementwise(golden):
    g = golden("elementwise")
    assert np.array_equal(O.relu_forward(g["x"]), g["relu_y"])
    assert np.array_equal(O.relu_backward(g["x"], g["dy"]), g["relu_dx"])
    assert O.rel_l2(O.leaky_relu_forward(g["x"]), g["lrelu_y"]) < 1e-6
    assert O.rel_l2(O.leaky_relu_backward(g["x"], g["dy"]), g["lrelu_dx"]) < 1e-6
    keep = (g["sd_mask"].ravel() > 0).astype(np.float64)
    y, mask = O.spatial_dropout_forward(g["x"], keep, 1 - float(g["sd_rate"]))
    assert O.rel_l2(y, g["sd_y"]) < 1e-7 and O.rel_l2(g["dy"] * mask, g["sd_dx"]) < 1e-7


def test_dense_loss_adam(golden):
    g = golden("dense_loss_adam")
    z = O.dense_forward(g["x"], g["w0"], g["b0"])
    assert O.rel_l2(z, g["z"]) < 1e-12
    p = O.softmax(z)
    assert O.rel_l2(p, g["p"]) < 1e-12
    assert O.rel_l2(O.cce_loss(p, g["labels"], 0.01, True), g["sample_losses"]) < 1e-12
    dz = O.softmax_cce_backward(p, g["labels"], 0.01)
    assert O.rel_l2(dz, g["dz"]) < 1e-7
    dx, dw, db = O.dense_backward(g["x"], g["w0"], g["b0"], dz, wl2=2e-5, bl2=1e-5)
    assert O.rel_l2(dx, g["dx"]) < 1e-7 and O.rel_l2(dw, g["dw"]) < 1e-7 and O.rel_l2(db, g["db"]) < 1e-7
    w, b = g["w0"], g["b0"]
    mw = vw = np.zeros_like(w); mb = vb = np.zeros_like(b)
    for it in range(3):
        lr = O.adam_lr(1e-3, 5e-5, it)
        assert np.isclose(lr, g["lrs"][it])
        w, mw, vw = O.adam_step(w, dw, mw, vw, lr, it)
        b, mb, vb = O.adam_step(b, db, mb, vb, lr, it)
        assert O.rel_l2(w, g["w_hist"][it]) < 1e-7 and O.rel_l2(b, g["b_hist"][it]) < 1e-7
    assert O.rel_l2(mw, g["m_w"]) < 1e-7 and O.rel_l2(vw, g["v_w"]) < 1e-7


def test_reference_checkpoint_format_loads_without_cupy(golden):
    """A parameter file in the reference CuPy model's on-disk format (pickled cupy arrays, CNN_model_cupy.py:277-282;
    the fixture was written by make_golden.py from the reference's NumPy model) unpickles to NumPy arrays through
    the restricted checkpoint unpickler; anything that is not an array constructor is refused."""
    import io
    import os
    import pickle

    from aether_ml_b200.model import _CheckpointUnpickler
    g = golden("checkpoint_cupy_format")
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "checkpoint_cupy_format.pkl")
    raw = open(path, "rb").read()
    assert b"cupy._core.core" in raw                       # the file really names cupy's constructor
    params = _CheckpointUnpickler(io.BytesIO(raw)).load()
    assert isinstance(params, list) and len(params) == 6
    assert [len(p) for p in params] == [2, 4, 2, 4, 2, 2]
    for k, layer_params in enumerate(params):
        for j, a in enumerate(layer_params):
            assert isinstance(a, np.ndarray)
            assert a.dtype == (np.float32 if k < 4 else np.float64)
            assert np.array_equal(a, g["p%d_%d" % (k, j)].astype(a.dtype))
    assert params[1][2].shape == (1, 1, 1, 4)              # keep-dims running statistics, as in the shipped files
    evil = pickle.dumps(os.system)                         # a global that is not an array constructor
    with pytest.raises(pickle.UnpicklingError):
        _CheckpointUnpickler(io.BytesIO(evil)).load()


def test_softmax_backward_matches_reference(golden):
    """The oracle's stand-alone SoftMax.backward against the array the reference's own Jacobian loop produced."""
    g = golden("softmax_backward")
    assert O.rel_l2(O.softmax(g["z"]), g["p"]) <= 1e-12
    assert O.rel_l2(O.softmax_backward(g["p"], g["dvalues"]), g["dinputs"]) <= 1e-12
    # the closed form the kernel uses: p * (dv - <p, dv>)
    p, dv = g["p"], g["dvalues"]
    closed = p * (dv - (p * dv).sum(axis=1, keepdims=True))
    assert O.rel_l2(closed, g["dinputs"]) <= 1e-12
