"""CPU oracle for the convolution hot path (TEST INFRASTRUCTURE, not product code).

A NumPy restatement of the arithmetic that Aether-ML's layer classes perform, written as
pure functions over arrays.  Only tests, the smoke check and the CPU-baseline leg of the
benchmark may import this module; the product path never does.

Each function names the reference lines whose arithmetic it restates (paths are relative
to the Aether-ML project root).  Parity of this module is pinned two ways:

* ``tests/golden/*.npz`` were produced by importing the reference's own NumPy classes
  (``CNN/models/CNN_classes.py``) and are compared with these functions in the CPU tests;
* the notebook known-answer values (``CNN/notebooks/CNN_Implementation.ipynb`` cells 8,
  14-16 and ``Backpropagation_Pooling.ipynb`` cells 0 and 6) are literal test vectors.

One deliberate difference: the reference's NumPy ``Conv_Layer.backward`` adds the
per-window contributions into an overlapping strided view, which under NumPy >= 1.13
keeps only the last writer.  The intended arithmetic -- the one its CuPy twin performs
with ``atomicAdd`` (``CNN/models/CNN_classes_cupy.py:4-35,141-146``) -- is a scatter-ADD,
and that is what :func:`conv_backward` computes.  :func:`conv_dinputs_last_writer`
reproduces the NumPy behaviour so the discrepancy stays on record.

All functions compute in float64 unless ``dtype`` says otherwise.
"""
from __future__ import annotations

import numpy as np
from numpy.lib.stride_tricks import sliding_window_view

__all__ = [
    "conv_out_hw", "conv_forward", "conv_backward", "conv_forward_blas", "conv_backward_blas",
    "conv_dinputs_last_writer", "bn_forward_train", "bn_forward_eval", "bn_backward",
    "pool_forward", "pool_backward", "relu_forward", "relu_backward", "leaky_relu_forward",
    "leaky_relu_backward", "spatial_dropout_forward", "dense_forward", "dense_backward",
    "softmax", "cce_loss", "softmax_cce_backward", "adam_step", "adam_lr", "rel_l2",
]


def rel_l2(a, b):
    """Relative L2 distance |a-b| / |b| in float64 (b is the oracle)."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    den = np.linalg.norm(b.ravel())
    num = np.linalg.norm((a - b).ravel())
    return float(num / den) if den > 0 else float(num)


# ----------------------------------------------------------------------------- convolution

def _pad_amount(filter_size, padding):
    # CNN_classes_cupy.py:78-81 -- 'same' pads (fH-1)//2 on BOTH axes, anything else pads 0.
    return (filter_size[0] - 1) // 2 if padding == "same" else 0


def conv_out_hw(H, W, filter_size, strides, padding):
    """Output height/width, CNN_classes_cupy.py:84-85 (int() of a float division)."""
    P = _pad_amount(filter_size, padding)
    Ho = int((H + 2 * P - filter_size[0]) / strides[0] + 1)
    Wo = int((W + 2 * P - filter_size[1]) / strides[1] + 1)
    return Ho, Wo


def _windows(xp, fH, fW, sH, sW, Ho, Wo):
    """(S,Ho,Wo,fH,fW,C) read-only window view of a padded NHWC array -- the same gather the
    reference builds with as_strided at CNN_classes_cupy.py:101-112."""
    v = sliding_window_view(xp, (fH, fW), axis=(1, 2))      # (S, H', W', C, fH, fW)
    v = v[:, ::sH, ::sW][:, :Ho, :Wo]
    return np.moveaxis(v, 3, 5)                                # (S, Ho, Wo, fH, fW, C)


def conv_forward(x, w, b, strides=(1, 1), padding="same", dtype=np.float64):
    """y[s,h,w,d] = sum_{i,j,c} xpad[s,h*sH+i,w*sW+j,c] * w[i,j,c,d] + b[d].

    Restates Conv_Layer.forward, CNN_classes_cupy.py:70-120 (NumPy twin CNN_classes.py:32-82):
    zero padding (:92-95), window gather (:101-112), einsum contraction (:115), bias (:116).
    x is NHWC, w is (fH,fW,Cin,Cout)."""
    x = np.asarray(x, dtype=dtype)
    w = np.asarray(w, dtype=dtype)
    fH, fW = w.shape[:2]
    sH, sW = strides
    P = _pad_amount((fH, fW), padding)
    Ho, Wo = conv_out_hw(x.shape[1], x.shape[2], (fH, fW), strides, padding)
    xp = np.pad(x, ((0, 0), (P, P), (P, P), (0, 0)))
    win = _windows(xp, fH, fW, sH, sW, Ho, Wo)
    y = np.einsum("shwxyc,xycd->shwd", win, w)
    return y + np.asarray(b, dtype=dtype).reshape(1, 1, 1, -1)


def conv_backward(x, w, dy, strides=(1, 1), padding="same", dtype=np.float64):
    """Returns (dx, dw, db) of Conv_Layer.backward, CNN_classes_cupy.py:123-154.

    db = sum of dy over (s,h,w) (:132); dw = windows^T . dy (:134); the per-window
    contributions dy . w^T (:138) are scatter-ADDED into the padded input gradient
    (kernel :16-32) and the padding border is cut off again (:149-153)."""
    x = np.asarray(x, dtype=dtype)
    w = np.asarray(w, dtype=dtype)
    dy = np.asarray(dy, dtype=dtype)
    fH, fW, Cin, Cout = w.shape
    sH, sW = strides
    P = _pad_amount((fH, fW), padding)
    S, H, W_, _ = x.shape
    _, Ho, Wo, _ = dy.shape
    xp = np.pad(x, ((0, 0), (P, P), (P, P), (0, 0)))
    win = _windows(xp, fH, fW, sH, sW, Ho, Wo)
    db = dy.sum(axis=(0, 1, 2))
    dw = np.einsum("shwxyc,shwd->xycd", win, dy)
    contrib = np.einsum("shwd,xycd->shwxyc", dy, w)
    dxp = np.zeros_like(xp)
    for i in range(fH):
        for j in range(fW):
            dxp[:, i:i + (Ho - 1) * sH + 1:sH, j:j + (Wo - 1) * sW + 1:sW, :] += contrib[:, :, :, i, j, :]
    dx = dxp[:, P:P + H, P:P + W_, :]
    return np.ascontiguousarray(dx), dw, db


def conv_dinputs_last_writer(x, w, dy, strides=(1, 1), padding="same"):
    """What the reference's NumPy Conv_Layer.backward actually returns for dinputs
    (CNN_classes.py:102-116): the in-place add on an overlapping view is executed on a
    temporary and copied back, so of the up-to fH*fW contributions per cell only the one
    written last (largest window index in C order) survives.  Kept for the record only."""
    x = np.asarray(x, dtype=np.float64)
    w = np.asarray(w, dtype=np.float64)
    dy = np.asarray(dy, dtype=np.float64)
    fH, fW, Cin, Cout = w.shape
    sH, sW = strides
    P = _pad_amount((fH, fW), padding)
    S, H, W_, _ = x.shape
    _, Ho, Wo, _ = dy.shape
    contrib = np.einsum("shwd,xycd->shwxyc", dy, w)
    dxp = np.zeros((S, H + 2 * P, W_ + 2 * P, Cin))
    # C-order traversal of (h, w, i, j): later assignments overwrite earlier ones.
    for h in range(Ho):
        for ww in range(Wo):
            dxp[:, h * sH:h * sH + fH, ww * sW:ww * sW + fW, :] = contrib[:, h, ww]
    return dxp[:, P:P + H, P:P + W_, :]


def conv_forward_blas(x, w, b, strides=(1, 1), padding="same", dtype=np.float32):
    """Same contraction as :func:`conv_forward`, evaluated tap by tap with matrix products
    (multi-threaded BLAS).  Used where the einsum form is too slow (full-size checks) and as
    the fairness footnote of the CPU baseline; cross-checked against conv_forward in tests."""
    x = np.asarray(x, dtype=dtype)
    w = np.asarray(w, dtype=dtype)
    fH, fW, Cin, Cout = w.shape
    sH, sW = strides
    P = _pad_amount((fH, fW), padding)
    Ho, Wo = conv_out_hw(x.shape[1], x.shape[2], (fH, fW), strides, padding)
    xp = np.pad(x, ((0, 0), (P, P), (P, P), (0, 0)))
    S = x.shape[0]
    y = np.zeros((S * Ho * Wo, Cout), dtype=dtype)
    for i in range(fH):
        for j in range(fW):
            a = xp[:, i:i + (Ho - 1) * sH + 1:sH, j:j + (Wo - 1) * sW + 1:sW, :]
            y += a.reshape(-1, Cin) @ w[i, j]
    return y.reshape(S, Ho, Wo, Cout) + np.asarray(b, dtype=dtype).reshape(1, 1, 1, -1)


def conv_backward_blas(x, w, dy, strides=(1, 1), padding="same", dtype=np.float32):
    """Tap-by-tap matrix-product evaluation of :func:`conv_backward` (same results up to
    rounding); see conv_forward_blas."""
    x = np.asarray(x, dtype=dtype)
    w = np.asarray(w, dtype=dtype)
    dy = np.asarray(dy, dtype=dtype)
    fH, fW, Cin, Cout = w.shape
    sH, sW = strides
    P = _pad_amount((fH, fW), padding)
    S, H, W_, _ = x.shape
    _, Ho, Wo, _ = dy.shape
    xp = np.pad(x, ((0, 0), (P, P), (P, P), (0, 0)))
    dxp = np.zeros_like(xp)
    dw = np.zeros_like(w)
    dy2 = dy.reshape(-1, Cout)
    for i in range(fH):
        for j in range(fW):
            sl = (slice(None), slice(i, i + (Ho - 1) * sH + 1, sH), slice(j, j + (Wo - 1) * sW + 1, sW), slice(None))
            a = xp[sl].reshape(-1, Cin)
            dw[i, j] = a.T @ dy2
            dxp[sl] += (dy2 @ w[i, j].T).reshape(S, Ho, Wo, Cin)
    db = dy2.sum(axis=0)
    return np.ascontiguousarray(dxp[:, P:P + H, P:P + W_, :]), dw, db


# ----------------------------------------------------------------------------- batch norm

def _bn_axes(x):
    return (0, 1, 2) if x.ndim == 4 else (0,)


def bn_forward_train(x, gamma, beta, running_mean, running_var, eps=1e-5, momentum=0.9, dtype=np.float64):
    """Batch_Norm.forward in training mode, CNN_classes_cupy.py:467-476: per-channel mean and
    BIASED variance over all axes but the last, eps inside the square root, running statistics
    updated as momentum*old + (1-momentum)*batch (with the biased variance).
    Returns (y, xhat, mean, var, new_running_mean, new_running_var); stats keep dims."""
    x = np.asarray(x, dtype=dtype)
    ax = _bn_axes(x)
    mean = x.mean(axis=ax, keepdims=True)
    var = x.var(axis=ax, keepdims=True)
    xhat = (x - mean) / np.sqrt(var + eps)
    y = np.asarray(gamma, dtype=dtype) * xhat + np.asarray(beta, dtype=dtype)
    rm = momentum * np.asarray(running_mean, dtype=dtype) + (1 - momentum) * mean
    rv = momentum * np.asarray(running_var, dtype=dtype) + (1 - momentum) * var
    return y, xhat, mean, var, rm, rv


def bn_forward_eval(x, gamma, beta, running_mean, running_var, eps=1e-5, dtype=np.float64):
    """Batch_Norm.forward with training=False, CNN_classes_cupy.py:478-480."""
    x = np.asarray(x, dtype=dtype)
    xhat = (x - np.asarray(running_mean, dtype=dtype)) / np.sqrt(np.asarray(running_var, dtype=dtype) + eps)
    return np.asarray(gamma, dtype=dtype) * xhat + np.asarray(beta, dtype=dtype)


def bn_backward(x, dy, gamma, mean, var, eps=1e-5, dtype=np.float64):
    """Batch_Norm.backward, CNN_classes_cupy.py:484-508, in the dvar/dmu form the reference
    uses.  Returns (dx, dgamma, dbeta)."""
    x = np.asarray(x, dtype=dtype)
    dy = np.asarray(dy, dtype=dtype)
    gamma = np.asarray(gamma, dtype=dtype)
    ax = _bn_axes(x)
    n = 1
    for a in ax:
        n *= x.shape[a]
    xc = x - mean
    inv = 1.0 / np.sqrt(var + eps)
    dxhat = dy * gamma
    dvar = np.sum(dxhat * xc * (-0.5) * np.power(var + eps, -1.5), axis=ax, keepdims=True)
    dmu = np.sum(-dxhat * inv, axis=ax, keepdims=True) + dvar * np.sum(-2.0 * xc, axis=ax, keepdims=True) / n
    dx = dxhat * inv + dvar * 2.0 * xc / n + dmu / n
    dgamma = np.sum(dy * (xc * inv), axis=ax)
    dbeta = np.sum(dy, axis=ax)
    return dx, dgamma, dbeta


# ----------------------------------------------------------------------------- pooling

def pool_forward(x, filter_size=(2, 2), strides=(2, 2), pooling_type="max", dtype=np.float64):
    """Pooling.forward with 'valid' padding, CNN_classes_cupy.py:212-273.  H_out =
    floor((H-f)/s + 1) (:223-224).  For max pooling also returns the window-local argmax
    (row, col) with the FIRST maximum in row-major window order (:259-265).
    Returns (y, (rows, cols)) for 'max' and (y, None) for 'average'."""
    x = np.asarray(x, dtype=dtype)
    fH, fW = filter_size
    sH, sW = strides
    S, H, W_, C = x.shape
    Ho = int(np.floor((H - fH) / sH + 1))
    Wo = int(np.floor((W_ - fW) / sW + 1))
    win = _windows(x, fH, fW, sH, sW, Ho, Wo)              # (S,Ho,Wo,fH,fW,C)
    if pooling_type == "max":
        flat = win.reshape(S, Ho, Wo, fH * fW, C)
        idx = flat.argmax(axis=3)
        y = np.take_along_axis(flat, idx[:, :, :, None, :], axis=3)[:, :, :, 0, :]
        return y, np.unravel_index(idx, (fH, fW))
    if pooling_type == "average":
        return win.mean(axis=(3, 4)), None
    raise ValueError(pooling_type)


def pool_backward(dy, in_shape, argmax=None, filter_size=(2, 2), strides=(2, 2), pooling_type="max",
                  dtype=np.float64):
    """Pooling.backward, CNN_classes_cupy.py:275-312: max pooling adds each dy to its window's
    argmax cell (:285-300, accumulating where windows overlap); average pooling adds
    dy/(fH*fW) to every cell of the window (:163-202)."""
    dy = np.asarray(dy, dtype=dtype)
    fH, fW = filter_size
    sH, sW = strides
    S, Ho, Wo, C = dy.shape
    dx = np.zeros(in_shape, dtype=dtype)
    if pooling_type == "max":
        rows, cols = argmax
        s_i, h_i, w_i, c_i = np.ogrid[:S, :Ho, :Wo, :C]
        np.add.at(dx, (s_i, h_i * sH + rows, w_i * sW + cols, c_i), dy)
    else:
        for i in range(fH):
            for j in range(fW):
                dx[:, i:i + (Ho - 1) * sH + 1:sH, j:j + (Wo - 1) * sW + 1:sW, :] += dy / (fH * fW)
    return dx


# ----------------------------------------------------------------------------- activations / dropout

def relu_forward(x):
    """ReLU.forward, CNN_classes_cupy.py:408-411."""
    return np.maximum(0, x)


def relu_backward(x, dy):
    """ReLU.backward, CNN_classes_cupy.py:413-415: gradient is zeroed where the INPUT is < 0
    (it passes at exactly 0)."""
    dx = np.array(dy, copy=True)
    dx[np.asarray(x) < 0] = 0
    return dx


def leaky_relu_forward(x, alpha=0.01):
    """Leaky_ReLU.forward, CNN_classes_cupy.py:421-424."""
    x = np.asarray(x)
    return np.where(x > 0, x, alpha * x)


def leaky_relu_backward(x, dy, alpha=0.01):
    """Leaky_ReLU.backward, CNN_classes_cupy.py:426-428 (scaled where input < 0)."""
    dx = np.array(dy, copy=True)
    dx[np.asarray(x) < 0] *= alpha
    return dx


def spatial_dropout_forward(x, channel_keep, keep_prob):
    """Layer_Dropout_Spatial.forward in training mode, CNN_classes_cupy.py:396-399, with the
    Bernoulli draw passed in (channel_keep in {0,1}, shape (C,)): one mask per channel shared
    by the whole batch, scaled by 1/keep_prob.  Backward multiplies dy by the same mask (:404).
    Returns (y, mask)."""
    mask = np.asarray(channel_keep, dtype=np.float64).reshape(1, 1, 1, -1) / keep_prob
    return np.asarray(x) * mask, mask


# ----------------------------------------------------------------------------- dense / softmax / loss

def dense_forward(x, w, b):
    """Layer_Dense.forward, CNN_classes_cupy.py:328-331."""
    return np.asarray(x, dtype=np.float64) @ np.asarray(w, dtype=np.float64) + np.asarray(b, dtype=np.float64)


def dense_backward(x, w, b, dy, wl1=0.0, wl2=0.0, bl1=0.0, bl2=0.0):
    """Layer_Dense.backward, CNN_classes_cupy.py:333-354, including the L1/L2 terms.
    Returns (dx, dw, db)."""
    x = np.asarray(x, dtype=np.float64)
    w = np.asarray(w, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    dy = np.asarray(dy, dtype=np.float64)
    dw = x.T @ dy
    db = dy.sum(axis=0, keepdims=True)
    if wl1 > 0:
        dw = dw + wl1 * np.where(w < 0, -1.0, 1.0)
    if wl2 > 0:
        dw = dw + 2 * wl2 * w
    if bl1 > 0:
        db = db + bl1 * np.where(b < 0, -1.0, 1.0)
    if bl2 > 0:
        db = db + 2 * bl2 * b
    return dy @ w.T, dw, db


def softmax(z):
    """SoftMax.forward, CNN_classes_cupy.py:542-547 (row max subtracted first)."""
    z = np.asarray(z, dtype=np.float64)
    e = np.exp(z - z.max(axis=1, keepdims=True))
    return e / e.sum(axis=1, keepdims=True)


def softmax_backward(p, dvalues):
    """SoftMax.backward, CNN_classes_cupy.py:549-560: per sample (diagflat(p) - p p^T) @ dvalues."""
    p = np.asarray(p, dtype=np.float64)
    dv = np.asarray(dvalues, dtype=np.float64)
    out = np.empty_like(dv)
    for i, (pi, di) in enumerate(zip(p, dv)):
        col = pi.reshape(-1, 1)
        out[i] = (np.diagflat(col) - col @ col.T) @ di
    return out


def _smooth_targets(y_true, n_classes, label_smoothing):
    y_true = np.asarray(y_true)
    if y_true.ndim == 1:
        y_true = np.eye(n_classes)[y_true]
    if label_smoothing > 0:
        y_true = y_true * (1.0 - label_smoothing) + label_smoothing / n_classes
    return y_true


def cce_loss(p, y_true, label_smoothing=0.0, training=True):
    """Per-sample loss of Loss_CategoricalCrossEntropy.forward, CNN_classes_cupy.py:615-632:
    probabilities clipped to [1e-7, 1-1e-7]; smoothing only when training."""
    p = np.asarray(p, dtype=np.float64)
    t = _smooth_targets(y_true, p.shape[1], label_smoothing if training else 0.0)
    return -np.sum(t * np.log(np.clip(p, 1e-7, 1 - 1e-7)), axis=1)


def softmax_cce_backward(p, y_true, label_smoothing=0.0):
    """Activation_Softmax_Loss_CategoricalCrossEntropy.backward, CNN_classes_cupy.py:666-680:
    (p - smoothed one-hot) / samples."""
    p = np.asarray(p, dtype=np.float64)
    t = _smooth_targets(y_true, p.shape[1], label_smoothing)
    return (p - t) / p.shape[0]


# ----------------------------------------------------------------------------- Adam

def adam_lr(learning_rate, decay, iterations):
    """Optimizer_Adam.pre_update_parameters, CNN_classes_cupy.py:695-701."""
    return learning_rate * (1.0 / (1.0 + decay * iterations)) if decay else learning_rate


def adam_step(p, g, m, v, lr, iterations, beta_1=0.9, beta_2=0.999, epsilon=1e-7):
    """One Optimizer_Adam.update_parameters for a single tensor, CNN_classes_cupy.py:710-734:
    bias correction uses iterations+1 and epsilon is added OUTSIDE the square root.
    Returns (p_new, m_new, v_new)."""
    p = np.asarray(p, dtype=np.float64)
    g = np.asarray(g, dtype=np.float64)
    m = beta_1 * np.asarray(m, dtype=np.float64) + (1 - beta_1) * g
    v = beta_2 * np.asarray(v, dtype=np.float64) + (1 - beta_2) * g * g
    mh = m / (1 - beta_1 ** (iterations + 1))
    vh = v / (1 - beta_2 ** (iterations + 1))
    return p - lr * mh / (np.sqrt(vh) + epsilon), m, v
