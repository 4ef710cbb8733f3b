"""Generate the golden fixtures in this directory by running Aether-ML's own NumPy classes.

Usage (needs a checkout of the reference project, which is NOT part of this repository):

    python tests/golden/make_golden.py /path/to/Aether-ML

Every array written here comes from executing ``CNN/models/CNN_classes.py`` unmodified on
seeded inputs, except ``conv_*/dx``: the reference's NumPy ``Conv_Layer.backward`` loses
all but one of the overlapping contributions (in-place add on an overlapping strided view),
so ``dx`` is built from the reference's own contributions tensor (its einsum at
``CNN_classes.py:98``) scatter-ADDED the way its CUDA kernel does
(``CNN_classes_cupy.py:16-32``); the verbatim NumPy result is kept as ``dx_verbatim``.
The notebook known-answer values are typed in from the stored cell outputs of
``CNN/notebooks/CNN_Implementation.ipynb`` (cells 8, 14, 15, 16).
"""
import os
import sys

import numpy as np


def main(ref_root):
    sys.path.insert(0, ref_root)
    from CNN.models import CNN_classes as R  # the reference's NumPy twin

    out_dir = os.path.dirname(os.path.abspath(__file__))
    rng = np.random.default_rng(20241)

    # ------------------------------------------------------------------ Conv_Layer cases
    conv_cases = {
        # name: (S, H, W, Cin, Cout, filter, strides, padding)
        "conv_same_3x3": (3, 6, 5, 3, 4, (3, 3), (1, 1), "same"),
        "conv_valid_3x3": (2, 7, 7, 2, 5, (3, 3), (1, 1), "valid"),
        "conv_same_5x5": (2, 8, 8, 3, 2, (5, 5), (1, 1), "same"),
        "conv_stride2_valid": (2, 9, 9, 2, 3, (3, 3), (2, 2), "valid"),
        "conv_tensor_path_small": (2, 8, 8, 64, 64, (3, 3), (1, 1), "same"),
        "conv_cfg1_tiny": (4, 32, 32, 3, 32, (3, 3), (1, 1), "same"),
    }
    for name, (S, H, W, Cin, Cout, f, st, pad) in conv_cases.items():
        np.random.seed(7)
        layer = R.Conv_Layer((H, W, Cin), num_filters=Cout, filter_size=f, strides=st, padding=pad)
        layer.biases = rng.standard_normal(Cout) * 0.1
        x = rng.random((S, H, W, Cin)).astype(np.float32)
        y = layer.forward(x.astype(np.float64), True)
        dy = rng.standard_normal(y.shape).astype(np.float32)
        dx_verbatim = np.array(layer.backward(dy.astype(np.float64)))
        # intended dX: the reference's own contributions, scatter-added
        contrib = np.einsum("shwd, xycd -> shwxyc", dy.astype(np.float64), layer.filter_weights)
        P = (f[0] - 1) // 2 if pad == "same" else 0
        dxp = np.zeros((S, H + 2 * P, W + 2 * P, Cin))
        Ho, Wo = y.shape[1:3]
        for i in range(f[0]):
            for j in range(f[1]):
                dxp[:, i:i + (Ho - 1) * st[0] + 1:st[0], j:j + (Wo - 1) * st[1] + 1:st[1], :] += contrib[:, :, :, i, j, :]
        dx = dxp[:, P:P + H, P:P + W, :]
        np.savez_compressed(
            os.path.join(out_dir, name + ".npz"),
            x=x, w=layer.filter_weights.astype(np.float32), b=layer.biases.astype(np.float32), dy=dy,
            y=y.astype(np.float32), dw=layer.dweights.astype(np.float32), db=layer.dbiases.astype(np.float32),
            dx=dx.astype(np.float32), dx_verbatim=dx_verbatim.astype(np.float32),
            strides=np.array(st), filter_size=np.array(f), padding=np.array(pad))

    # ------------------------------------------------------------------ Batch_Norm
    for name, shape in {"bn_4d": (4, 6, 6, 8), "bn_2d": (16, 12)}.items():
        bn = R.Batch_Norm(epsilon=1e-5, momentum=0.9)
        x = (rng.standard_normal(shape) * 2 + 0.5).astype(np.float32)
        y1 = np.array(bn.forward(x.astype(np.float64), True))          # creates gamma/beta/running stats
        bn.gamma[:] = rng.standard_normal(shape[-1]).astype(np.float32) + 1.0
        bn.beta[:] = rng.standard_normal(shape[-1]).astype(np.float32) * 0.1
        rm0 = np.array(bn.running_mean, dtype=np.float32)
        rv0 = np.array(bn.running_var, dtype=np.float32)
        y = np.array(bn.forward(x.astype(np.float64), True))
        dy = rng.standard_normal(shape).astype(np.float32)
        dx = np.array(bn.backward(dy.astype(np.float64)))
        y_eval = np.array(bn.forward(x.astype(np.float64), False))
        np.savez_compressed(
            os.path.join(out_dir, name + ".npz"), x=x, gamma=bn.gamma, beta=bn.beta, rm0=rm0, rv0=rv0,
            y=y.astype(np.float32), mean=np.array(bn.batch_mean, dtype=np.float32),
            var=np.array(bn.batch_var, dtype=np.float32), rm1=np.array(bn.running_mean, dtype=np.float32),
            rv1=np.array(bn.running_var, dtype=np.float32), dy=dy, dx=dx.astype(np.float32),
            dgamma=np.array(bn.dweights, dtype=np.float32), dbeta=np.array(bn.dbiases, dtype=np.float32),
            y_eval=y_eval.astype(np.float32), y_first=y1.astype(np.float32))

    # ------------------------------------------------------------------ Pooling
    pool_cases = {
        "pool_max_2x2": ((3, 8, 8, 5), (2, 2), (2, 2), "max"),
        "pool_max_odd": ((2, 7, 7, 3), (2, 2), (2, 2), "max"),
        "pool_max_overlap": ((2, 7, 6, 4), (3, 3), (2, 2), "max"),
        "pool_avg_2x2": ((2, 6, 6, 3), (2, 2), (2, 2), "average"),
    }
    for name, (shape, f, st, kind) in pool_cases.items():
        pool = R.Pooling(filter_size=f, strides=st, padding="valid", pooling_type=kind)
        x = rng.standard_normal(shape).astype(np.float32)
        if kind == "max":
            x[0, :2, :2, 0] = 0.0          # an all-equal window: first cell must win
            x = np.maximum(x, -0.3)        # plenty of ties at the floor value
        y = np.array(pool.forward(x, True))
        dy = rng.standard_normal(y.shape).astype(np.float32)
        dx = np.array(pool.backward(dy))
        extra = {}
        if kind == "max":
            extra = dict(arg_rows=np.array(pool.max_indicies[0]), arg_cols=np.array(pool.max_indicies[1]))
        np.savez_compressed(os.path.join(out_dir, name + ".npz"), x=x, y=y.astype(np.float32), dy=dy,
                            dx=dx.astype(np.float32), filter_size=np.array(f), strides=np.array(st),
                            kind=np.array(kind), **extra)

    # ------------------------------------------------------------------ ReLU / Leaky / spatial dropout
    x = rng.standard_normal((3, 4, 4, 6)).astype(np.float32)
    x[0, 0, 0, :3] = 0.0
    dy = rng.standard_normal(x.shape).astype(np.float32)
    relu = R.ReLU(); relu.forward(x, True); relu.backward(dy)
    lrelu = R.Leaky_ReLU(0.01); lrelu.forward(x, True); lrelu.backward(dy)
    np.random.seed(3)
    sd = R.Layer_Dropout_Spatial(0.3); sd.forward(x, True); sd.backward(dy)
    np.savez_compressed(os.path.join(out_dir, "elementwise.npz"), x=x, dy=dy,
                        relu_y=relu.output, relu_dx=relu.dinputs, lrelu_y=lrelu.output.astype(np.float32),
                        lrelu_dx=lrelu.dinputs, sd_mask=np.array(sd.channel_mask), sd_y=np.array(sd.output),
                        sd_dx=np.array(sd.dinputs), sd_rate=np.array(0.3))

    # ------------------------------------------------------------------ Dense + softmax/CCE + Adam
    np.random.seed(11)
    dense = R.Layer_Dense(12, 10, weight_regularizer_l2=2e-5, bias_regularizer_l2=1e-5)
    dense.weights = dense.weights * 100
    x = rng.standard_normal((8, 12)).astype(np.float32)
    labels = rng.integers(0, 10, 8)
    z = np.array(dense.forward(x.astype(np.float64), True))
    comb = R.Activation_Softmax_Loss_CategoricalCrossEntropy(label_smoothing=0.01)
    sm = R.SoftMax(); p = np.array(sm.forward(z, True))
    loss = R.Loss_CategoricalCrossEntropy(0.01)
    sample_losses = np.array(loss.forward(p, labels, True))
    comb.backward(p, labels, training=True)
    dz = np.array(comb.dinputs)
    dense.backward(dz)
    w0 = np.array(dense.weights); b0 = np.array(dense.biases)
    opt = R.Optimizer_Adam(learning_rate=1e-3, decay=5e-5)
    hist_w, hist_b, lrs = [], [], []
    for _ in range(3):
        opt.pre_update_parameters()
        opt.update_parameters(dense)
        opt.post_update_parameters()
        hist_w.append(np.array(dense.weights)); hist_b.append(np.array(dense.biases)); lrs.append(opt.current_learning_rate)
    np.savez_compressed(os.path.join(out_dir, "dense_loss_adam.npz"), x=x, labels=labels, w0=w0, b0=b0, z=z, p=p,
                        sample_losses=sample_losses, dz=dz, dw=np.array(dense.dweights), db=np.array(dense.dbiases),
                        dx=np.array(dense.dinputs), w_hist=np.stack(hist_w), b_hist=np.stack(hist_b),
                        lrs=np.array(lrs), m_w=np.array(dense.weight_momentums), v_w=np.array(dense.weight_cache))

    # ------------------------------------------------------------------ SoftMax.backward on its own (the Jacobian loop)
    sm = R.SoftMax()
    zs = rng.standard_normal((7, 10)) * 2.0
    ps = sm.forward(zs, True)
    dvs = rng.standard_normal((7, 10))
    sm.backward(dvs)
    np.savez_compressed(os.path.join(out_dir, "softmax_backward.npz"), z=zs, p=np.array(ps), dvalues=dvs,
                        dinputs=np.array(sm.dinputs))

    # ------------------------------------------------------------------ notebook known answers
    np.savez_compressed(
        os.path.join(out_dir, "notebook_kat.npz"),
        image=np.array([[1, 2, 3, 0], [0, 1, 2, 3], [3, 0, 1, 2], [2, 3, 0, 1]], dtype=np.float32),
        kernel=np.array([[1, 0, -1], [1, 0, -1], [1, 0, -1]], dtype=np.float32),
        expected=np.array([[-3, -4, 0, 5], [-3, -2, -2, 6], [-4, 2, -2, 3], [-3, 4, 0, 1]], dtype=np.float32))
    # ------------------------------------------------------------------ parameter checkpoint in the CuPy model's format
    # A small network in the layout of the reference's shipped checkpoints (CNN/saved_models/model2..5: conv, BN,
    # conv, BN, ..., dense, dense; float32 conv/BN arrays with keep-dims running statistics, float64 dense arrays),
    # built and evaluated with the reference's NumPy Model.  The file is written the way the CuPy model writes it
    # (CNN_model_cupy.py:277-282): every array pickles as a call of ``cupy._core.core.array`` on its host copy,
    # which is what ``cupy.ndarray.__reduce__`` emits.  CuPy itself is not needed: a stand-in module of that name
    # provides the constructor while the file is being written.
    import pickle
    import types
    from CNN.models import CNN_model as RM
    np.random.seed(11)
    net = RM.Model()
    net.add(R.Conv_Layer((8, 8, 1), num_filters=4, filter_size=(3, 3), strides=(1, 1), padding="same"))
    net.add(R.Batch_Norm())
    net.add(R.ReLU())
    net.add(R.Pooling((2, 2), (2, 2), "valid", "max"))
    net.add(R.Conv_Layer((4, 4, 4), num_filters=8, filter_size=(3, 3), strides=(1, 1), padding="same"))
    net.add(R.Batch_Norm())
    net.add(R.ReLU())
    net.add(R.Pooling((2, 2), (2, 2), "valid", "max"))
    net.add(R.Flatten())
    net.add(R.Layer_Dense(2 * 2 * 8, 12))
    net.add(R.ReLU())
    net.add(R.Layer_Dense(12, 5))
    net.add(R.SoftMax())
    net.set(loss=R.Loss_CategoricalCrossEntropy(), optimizer=R.Optimizer_Adam(learning_rate=1e-2),
            accuracy=RM.Accuracy_Categorical())
    for layer in net.layers:                             # the CuPy twin's alias (CNN_classes_cupy.py:68): conv layers train
        if isinstance(layer, R.Conv_Layer):
            layer.weights = layer.filter_weights
    net.finalize()
    xs = rng.random((6, 8, 8, 1)).astype(np.float32)
    ys = rng.integers(0, 5, size=6)
    for _ in range(3):                                   # a few steps so that no parameter is at its initial value
        out = net.forward(xs.astype(np.float64), training=True)
        net.backward(out, ys)
        net.optimizer.pre_update_parameters()
        for layer in net.trainable_layers:
            net.optimizer.update_parameters(layer)
        net.optimizer.post_update_parameters()
    probs = net.forward(xs.astype(np.float64), training=False)
    # per-layer tuples as the CuPy twin's get_parameters returns them (the NumPy Batch_Norm has no such method):
    # conv (filter_weights, biases) CNN_classes_cupy.py:156-158, Batch_Norm (gamma, beta, running_mean, running_var)
    # :510-516 with (C,) parameters and keep-dims statistics as in the shipped checkpoints, dense (weights, biases)
    params = []
    for layer in (l for l in net.layers if isinstance(l, (R.Conv_Layer, R.Batch_Norm, R.Layer_Dense))):
        if isinstance(layer, R.Batch_Norm):
            Cn = np.asarray(layer.gamma).size
            params.append((np.asarray(layer.gamma).reshape(-1), np.asarray(layer.beta).reshape(-1),
                           np.asarray(layer.running_mean).reshape(1, 1, 1, Cn),
                           np.asarray(layer.running_var).reshape(1, 1, 1, Cn)))
        elif isinstance(layer, R.Conv_Layer):
            params.append((np.asarray(layer.filter_weights), np.asarray(layer.biases)))
        else:
            params.append((np.asarray(layer.weights), np.asarray(layer.biases)))

    stub_names = ("cupy", "cupy._core", "cupy._core.core")
    saved_modules = {n: sys.modules.get(n) for n in stub_names}
    mods = {n: types.ModuleType(n) for n in stub_names}

    def array(host):
        return np.asarray(host)
    array.__module__ = "cupy._core.core"
    array.__qualname__ = "array"
    mods["cupy._core.core"].array = array
    mods["cupy._core"].core = mods["cupy._core.core"]
    mods["cupy"]._core = mods["cupy._core"]

    class DeviceArray:                                   # pickles like cupy.ndarray: array(host copy)
        def __init__(self, host):
            self.host = host

        def __reduce__(self):
            return array, (self.host,)

    def as_saved(a, k):
        a = np.asarray(a)
        # conv and BN arrays are float32 in the CuPy model (CNN_classes_cupy.py:44,66,443-448), dense ones float64
        return DeviceArray(a.astype(np.float32) if k < 4 else a.astype(np.float64))

    sys.modules.update(mods)
    try:
        with open(os.path.join(out_dir, "checkpoint_cupy_format.pkl"), "wb") as fh:
            pickle.dump([tuple(as_saved(a, k) for a in layer_params) for k, layer_params in enumerate(params)], fh)
    finally:
        for n, m in saved_modules.items():
            if m is None:
                sys.modules.pop(n, None)
            else:
                sys.modules[n] = m
    np.savez_compressed(os.path.join(out_dir, "checkpoint_cupy_format.npz"), x=xs, probs=probs.astype(np.float64),
                        **{"p%d_%d" % (k, j): np.asarray(a) for k, lp in enumerate(params) for j, a in enumerate(lp)})
    print("golden fixtures written to", out_dir)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
