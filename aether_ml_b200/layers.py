"""Layer, loss and optimizer classes with the names, constructor arguments, methods and attributes of
Aether-ML's ``CNN/models/CNN_classes_cupy.py``, computing on a B200 through libaether_b200.so.

Every ``forward`` / ``backward`` below is a thin host-side wrapper: it validates shapes, owns the
output / workspace buffers (torch CUDA tensors are used purely as device memory) and makes one or
two C-ABI calls.  No arithmetic on activations happens in Python and there is no CPU fallback.

Arrays: fp32, C-contiguous, NHWC activations, (fH, fW, Cin, Cout) filters -- the reference's layouts.
Inputs may be torch CUDA tensors, objects exposing ``__cuda_array_interface__`` (CuPy arrays) or
NumPy arrays (copied to the device).  Outputs are torch CUDA tensors.
"""
import ctypes as C
import os

import numpy as np
import torch

from . import _lib
from ._lib import AetherConvDesc, check, lib

DEFAULT_MATH_MODE = os.environ.get("AETHER_MATH_MODE", "bf16")


def _device():
    if not torch.cuda.is_available():
        raise _lib.AetherError("aether_ml_b200 needs a CUDA device (no CPU fallback exists)")
    return torch.device("cuda", torch.cuda.current_device())


def to_device(a, dtype=torch.float32):
    """Return `a` as a contiguous CUDA tensor of `dtype` (no copy when it already is one)."""
    if isinstance(a, torch.Tensor):
        t = a
    elif hasattr(a, "__cuda_array_interface__"):
        t = torch.as_tensor(a, device=_device())
    else:
        t = torch.as_tensor(np.asarray(a))
    if t.device.type != "cuda":
        t = t.to(_device(), non_blocking=True)
    if t.dtype != dtype:
        t = t.to(dtype)
    return t if t.is_contiguous() else t.contiguous()


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _empty(shape, dtype=torch.float32):
    return torch.empty(shape, dtype=dtype, device=_device())


class _Saved:
    """Pickling of a layer / loss / optimizer for ``Model.save`` (the reference pickles the whole model after
    stripping the per-step arrays, CNN_model_cupy.py:291-309): device arrays travel as NumPy arrays, everything that
    belongs to one forward/backward pass (activations, gradients, workspaces, operand-copy bookkeeping, links to the
    neighbouring layers) is left out and rebuilt empty on loading."""

    _TRANSIENT = ("inputs", "output", "dinputs", "dweights", "dbiases", "prev", "next", "bn_partials", "binary_mask",
                  "channel_mask", "batch_mean", "batch_var", "running_mean", "running_var", "inputs_shape",
                  "trainable_layers", "accumulated_sum", "accumulated_count", "step_dev", "stats_from", "fused_dropout",
                  "fused_pool", "fused_bn", "copy_consumer", "copy_dy_consumer", "fixed_mask", "fused_into_prev")

    def __getstate__(self):
        state = {}
        for k, v in self.__dict__.items():
            if k in self._TRANSIENT or (k.startswith("_") and k not in ("_rm", "_rv", "_calls")):
                continue
            state[k] = ("__device_array__", v.detach().cpu().numpy()) if isinstance(v, torch.Tensor) else v
        return state

    def __setstate__(self, state):
        for k, v in state.items():
            if isinstance(v, tuple) and len(v) == 2 and isinstance(v[0], str) and v[0] == "__device_array__":
                v = to_device(v[1], torch.from_numpy(v[1]).dtype)
            self.__dict__[k] = v
        self._restore_transient()

    def _restore_transient(self):
        pass


class _Workspace:
    """Grow-only byte buffer owned by a layer and handed to the library as scratch."""

    def __init__(self):
        self.buf = None

    def get(self, nbytes):
        nbytes = max(int(nbytes), 256)
        if self.buf is None or self.buf.numel() < nbytes:
            self.buf = torch.empty(nbytes, dtype=torch.uint8, device=_device())
        return self.buf


class _OperandCopies:
    """Remembers which arrays the forward pass left bf16 operand copies of in a layer's workspace, so that the
    backward pass reuses a copy only while it still describes the array: same workspace buffer, same array, and
    no in-place change since (torch's per-tensor version counter).  Anything else -- a regrown workspace, an input
    modified between the passes, weights replaced -- makes the backward pass rebuild the copy."""

    def __init__(self):
        self.ws_ptr = None
        self.x = None
        self.w = None

    @staticmethod
    def _tag(t):
        return (t.data_ptr(), t._version, tuple(t.shape))

    def record(self, ws, x, w):
        self.ws_ptr = ws.data_ptr()
        self.x = self._tag(x)
        self.w = self._tag(w)

    def flags(self, ws, x, w):
        """Bit 0: the copy of x is valid; bit 1: the copies of the weights are (aether_conv2d_bwd's x_shadow_valid)."""
        if self.ws_ptr is None or ws.data_ptr() != self.ws_ptr:
            return 0
        return (1 if self._tag(x) == self.x else 0) | (2 if self._tag(w) == self.w else 0)


def _mark_unwritten(t):
    """Marks a device array whose fp32 contents were deliberately not written (lean mode: only its bf16 operand copy
    exists, inside the consuming layer's workspace).  A layer that would have to READ such an array raises."""
    t._aether_unwritten = True
    return t


def _require_written(t, who):
    if getattr(t, "_aether_unwritten", False):
        raise _lib.AetherError("%s: the input array was not materialised (Model.finalize(lean=True)) and its operand copy is "
                               "no longer current; run the producing layer again" % who)


def _array_tag(t):
    """Identity of a device array's contents as far as the host can tell: address, element count, version counter
    (a reshaped view of the same memory has the same tag)."""
    return (t.data_ptr(), t.numel(), t._version)


class _HandedIn:
    """Operand copies that a neighbouring layer's kernel wrote into this layer's workspace (see
    aether_conv2d_operand_layout): which array each describes, so the layer skips its own cast pass only for
    exactly that array in exactly that workspace buffer."""

    def __init__(self):
        self.x = None        # (workspace address, tag of x)
        self.dy = None       # (workspace address, tag of dy, rows of column sums)

    def x_ready(self, ws, x):
        return self.x is not None and self.x == (ws.data_ptr(), _array_tag(x))

    def dy_rows(self, ws, dy):
        if self.dy is not None and self.dy[:2] == (ws.data_ptr(), _array_tag(dy)):
            return self.dy[2]
        return 0


def _operand_layout(d):
    """AetherOperandLayout of a convolution descriptor, or None when the shape reads no bf16 operand copies."""
    lay = _lib.AetherOperandLayout()
    return lay if lib().aether_conv2d_operand_layout(C.byref(d), C.byref(lay)) else None


# ------------------------------------------------------------------------------------- Conv_Layer
class Conv_Layer(_Saved):
    """Drop-in for ``Conv_Layer`` (CNN_classes_cupy.py:37-161).

    Same constructor arguments and attributes (``filter_weights``/``weights`` alias, ``biases``, the
    four regularizer attributes; after ``forward``: ``output``, ``inputs``; after ``backward``:
    ``dweights``, ``dbiases``, ``dinputs``).  ``dinputs`` is the scatter-ADD gradient that the
    reference's CUDA scatter kernel produces (:4-35), returned contiguous instead of as a sliced view.
    One extra keyword, ``math_mode`` in {"bf16", "tf32", "fp32"}, selects the operand precision of
    the tensor-core kernels (default from $AETHER_MATH_MODE, else bf16)."""

    def __init__(self, input_shape, num_filters=1, filter_size=(3, 3), strides=(1, 1), padding="same",
                 math_mode=None):
        self.input_shape = input_shape
        self.num_filters = num_filters
        self.filter_size = filter_size
        self.strides = strides
        self.padding = padding
        self.math_mode = math_mode or DEFAULT_MATH_MODE
        if self.math_mode not in _lib.MATH_MODES:
            raise ValueError("math_mode must be one of %s" % sorted(_lib.MATH_MODES))
        self.weight_regularizer_l1 = 0
        self.weight_regularizer_l2 = 0
        self.bias_regularizer_l1 = 0
        self.bias_regularizer_l2 = 0
        input_depth = input_shape[-1]
        n = filter_size[0] * filter_size[1] * input_depth
        std = np.float32(np.sqrt(np.float32(2.0 / n)))
        # He-normal initialisation (:54-66), drawn on the host from NumPy's global generator
        w = np.random.randn(filter_size[0], filter_size[1], input_depth, num_filters).astype(np.float32) * std
        self.filter_weights = to_device(w)
        self.biases = torch.zeros(num_filters, dtype=torch.float32, device=_device())
        self._ws = _Workspace()
        self._stats_ws = _Workspace()
        self.emit_bn_stats = False      # set when a Batch_Norm consumes this layer's output (Model.finalize does it)
        self.bn_partials = None         # (buffer, blocks, data_ptr of the output they describe) after a training forward
        self._desc = None
        self._copies = _OperandCopies()
        self._handed = _HandedIn()
        self.first_in_model = False     # Model.finalize: this layer's dinputs are never needed

    def _restore_transient(self):
        self._ws = _Workspace()
        self._stats_ws = _Workspace()
        self.bn_partials = None
        self._desc = None
        self._copies = _OperandCopies()
        self._handed = _HandedIn()
        self.emit_bn_stats = False
        self.first_in_model = False

    # `weights` is the same array object as `filter_weights` (:68); in-place optimizer updates on
    # either name are visible through both.
    @property
    def weights(self):
        return self.filter_weights

    @weights.setter
    def weights(self, value):
        self.filter_weights = value

    def _make_desc(self, S, H, W, Cin):
        fH, fW = self.filter_size
        sH, sW = self.strides
        P = (fH - 1) // 2 if self.padding == "same" else 0      # :78-81, same amount on both axes
        Ho = int((H + 2 * P - fH) / sH + 1)
        Wo = int((W + 2 * P - fW) / sW + 1)
        d = AetherConvDesc(S, H, W, Cin, self.num_filters, fH, fW, sH, sW, P, P, _lib.MATH_MODES[self.math_mode])
        return d, Ho, Wo

    # -- operand-copy hand-off: the kernel that produces this layer's x (going forward) or dy (going back) may write
    # the bf16 copy the tensor-core kernels read straight into this layer's workspace
    def x_copy_target(self, shape):
        """(address, row length) where the bf16 copy of an input of `shape` goes, or None."""
        if len(shape) != 4 or shape[3] != self.filter_weights.shape[2]:
            return None
        d, Ho, Wo = self._make_desc(*shape)
        lay = _operand_layout(d) if (Ho >= 1 and Wo >= 1) else None
        if lay is None or lay.x_copy_ld == 0:          # (first layers gather x themselves: no copy of x is read)
            return None
        ws = self._ws.get(lib().aether_conv2d_workspace_bytes(C.byref(d)))
        return ws.data_ptr() + lay.x_copy_offset, lay.x_copy_ld

    def x_copy_written(self, x):
        self._handed.x = (self._ws.buf.data_ptr(), _array_tag(x))

    def dy_copy_target(self):
        """(address, row length, column-sum address, rows available) for the bf16 copy of the coming dvalues, or None."""
        if self._desc is None:
            return None
        lay = _operand_layout(self._desc)
        if lay is None:
            return None
        # A first layer's filter-gradient kernel takes the copy, but its dX runs on the CUDA cores from the fp32 array:
        # the hand-off is only for a layer whose dinputs nobody asks for (the first layer of a Model).
        if lay.x_copy_ld == 0 and not self.first_in_model:
            return None
        ws = self._ws.get(lib().aether_conv2d_workspace_bytes(C.byref(self._desc)))
        return ws.data_ptr() + lay.dy_copy_offset, lay.dy_copy_ld, ws.data_ptr() + lay.dy_colsum_offset, lay.dy_colsum_rows_max

    def dy_copy_written(self, dy, rows):
        self._handed.dy = (self._ws.buf.data_ptr(), _array_tag(dy), int(rows))

    def forward(self, inputs, training):
        x = to_device(inputs)
        if x.ndim != 4:
            raise ValueError(f"Expected a 4D tensor, got {x.ndim} instead.")
        S, H, W, Cin = x.shape
        if Cin != self.filter_weights.shape[2]:
            raise ValueError(f"input has {Cin} channels, filters expect {self.filter_weights.shape[2]}")
        d, Ho, Wo = self._make_desc(S, H, W, Cin)
        if Ho < 1 or Wo < 1:
            raise ValueError("filter larger than the padded input")
        L = lib()
        ws = self._ws.get(L.aether_conv2d_workspace_bytes(C.byref(d)))
        y = _empty((S, Ho, Wo, self.num_filters))
        flags = _lib.CONV_X_COPY_READY if self._handed.x_ready(ws, x) else 0
        self._handed.x = None
        if not flags:
            _require_written(x, "Conv_Layer.forward")
        # With emit_bn_stats the kernel's epilogue also writes the per-channel partial statistics that the
        # Batch_Norm behind this layer would otherwise compute in a pass of its own over y (:467-470).
        nblk = int(L.aether_conv2d_bnstats_blocks(C.byref(d))) if (training and self.emit_bn_stats) else 0
        self.bn_partials = None
        if nblk > 0:
            stats = self._stats_ws.get(nblk * 3 * self.num_filters * 4)
            check(L.aether_conv2d_fwd_ex(C.byref(d), _ptr(x), _ptr(self.filter_weights), _ptr(self.biases), _ptr(y),
                                         _ptr(stats), stats.numel(), _ptr(ws), ws.numel(), flags, _stream()),
                  "aether_conv2d_fwd_ex")
            self.bn_partials = (stats, nblk, y.data_ptr())
        else:
            check(L.aether_conv2d_fwd_ex(C.byref(d), _ptr(x), _ptr(self.filter_weights), _ptr(self.biases), _ptr(y),
                                         None, 0, _ptr(ws), ws.numel(), flags, _stream()), "aether_conv2d_fwd_ex")
        self.inputs = x
        self.output = y
        self._desc = d
        self._copies.record(ws, x, self.filter_weights)
        return self.output

    def backward(self, dvalues, need_dinputs=True):
        if self._desc is None:
            raise RuntimeError("Conv_Layer.backward called before forward")
        dy = to_device(dvalues)
        d = self._desc
        x = self.inputs
        Ho = (d.H + 2 * d.padH - d.fH) // d.sH + 1
        Wo = (d.W + 2 * d.padW - d.fW) // d.sW + 1
        if tuple(dy.shape) != (d.S, Ho, Wo, d.Cout):
            raise ValueError(f"dvalues has shape {tuple(dy.shape)}, expected {(d.S, Ho, Wo, d.Cout)}")
        L = lib()
        ws = self._ws.get(L.aether_conv2d_workspace_bytes(C.byref(d)))
        if getattr(self, "_grad_views", None) is not None:
            self.dweights, self.dbiases = self._grad_views
        else:
            self.dweights = _empty(tuple(self.filter_weights.shape))
            self.dbiases = _empty((d.Cout,))
        dx = _empty((d.S, d.H, d.W, d.Cin)) if need_dinputs else None
        shadow_ok = self._copies.flags(ws, x, self.filter_weights)
        rows = self._handed.dy_rows(ws, dy)
        self._handed.dy = None
        if rows and self.first_in_model and need_dinputs:
            rows = 0                        # a first layer asked for dinputs after all: that path reads the fp32 array
        if rows:
            shadow_ok |= _lib.CONV_DY_COPY_READY
        else:
            _require_written(dy, "Conv_Layer.backward")
        if not (shadow_ok & _lib.CONV_X_COPY_READY) and self.dweights is not None:
            _require_written(x, "Conv_Layer.backward")
        check(L.aether_conv2d_bwd_ex(C.byref(d), _ptr(x), _ptr(dy), _ptr(self.filter_weights), _ptr(dx),
                                     _ptr(self.dweights), _ptr(self.dbiases), _ptr(ws), ws.numel(), shadow_ok, rows,
                                     _stream()), "aether_conv2d_bwd_ex")
        self.dinputs = dx
        return self.dinputs

    def get_parameters(self):
        return self.filter_weights, self.biases

    def set_parameters(self, weights, biases):
        # copy into the existing arrays so `weights` stays the same object as `filter_weights`
        w = to_device(weights)
        b = to_device(biases).reshape(-1)
        if tuple(w.shape) != tuple(self.filter_weights.shape) or b.numel() != self.biases.numel():
            raise ValueError("parameter shapes do not match this layer")
        self.filter_weights.copy_(w)
        self.biases.copy_(b)


# ------------------------------------------------------------------------------------- Pooling
class Pooling(_Saved):
    """Drop-in for ``Pooling`` (CNN_classes_cupy.py:204-312), 'valid' padding, max or average.
    The argmax is kept as one byte per output (window-local index of the first maximum);
    ``max_indicies`` reconstructs the reference's (rows, cols) pair on demand."""

    def __init__(self, filter_size=(2, 2), strides=(2, 2), padding="valid", pooling_type="max"):
        self.filter_size = filter_size
        self.strides = strides
        self.padding = padding
        self.pooling_type = pooling_type
        self.fused_bn = None            # a Batch_Norm that pools inside its own kernels (Model.finalize(fuse=True))

    def _restore_transient(self):
        self.fused_bn = None

    def _kind(self):
        if self.pooling_type == "max":
            return _lib.POOL_MAX
        if self.pooling_type == "average":
            return _lib.POOL_AVG
        raise ValueError(f"Expected pooling_type == max or average, recieved {self.pooling_type} instead")

    def forward(self, inputs, training):
        x = to_device(inputs)
        if self.fused_bn is not None and self.fused_bn.pooled_now:
            # the fused Batch_Norm already produced the pooled tensor (and keeps the argmax codes)
            self.inputs = self.output = x
            self._argmax = self.fused_bn._pool_arg
            return self.output
        if x.ndim != 4:
            raise ValueError(f"Expected a 4D tensor, got {x.ndim} instead.")
        if self.padding != "valid":
            # the reference's "same" branch reads H_out before assigning it (:226-233) and cannot run
            raise ValueError(f"Expected padding == valid, recieved {self.padding} instead")
        S, H, W, Cc = x.shape
        fH, fW = self.filter_size
        sH, sW = self.strides
        Ho = (H - fH) // sH + 1
        Wo = (W - fW) // sW + 1
        kind = self._kind()
        y = _empty((S, Ho, Wo, Cc))
        self._argmax = _empty((S, Ho, Wo, Cc), torch.uint8) if kind == _lib.POOL_MAX else None
        check(lib().aether_pool_fwd(_ptr(x), _ptr(y), _ptr(self._argmax), S, H, W, Cc, fH, fW, sH, sW, kind,
                                    _stream()), "aether_pool_fwd")
        self.inputs = x
        self.output = y
        return self.output

    @property
    def max_indicies(self):
        fW = self.filter_size[1]
        code = self._argmax.to(torch.int64)
        return code // fW, code % fW

    def backward(self, dvalues):
        dy = to_device(dvalues)
        if self.fused_bn is not None and self.fused_bn.pooled_now:
            self.dinputs = dy
            return self.dinputs
        S, H, W, Cc = self.inputs.shape
        fH, fW = self.filter_size
        sH, sW = self.strides
        dx = _empty((S, H, W, Cc))
        check(lib().aether_pool_bwd(_ptr(dy), _ptr(self._argmax), _ptr(dx), S, H, W, Cc, fH, fW, sH, sW,
                                    self._kind(), _stream()), "aether_pool_bwd")
        self.dinputs = dx
        return self.dinputs


# ------------------------------------------------------------------------------------- activations
class ReLU(_Saved):
    """Drop-in for ``ReLU`` (CNN_classes_cupy.py:406-415).  With ``fused_into_prev`` (set by
    ``Model.finalize(fuse=True)`` when the layer follows a Batch_Norm) the activation is applied by that
    Batch_Norm's kernels and this layer only hands tensors through."""
    _alpha = 0.0
    fused_into_prev = False

    def forward(self, inputs, training):
        x = to_device(inputs)
        if self.fused_into_prev:
            self.inputs = self.output = x
            return self.output
        y = torch.empty_like(x)
        check(lib().aether_leaky_relu_fwd(_ptr(x), _ptr(y), x.numel(), float(self._alpha), _stream()),
              "aether_leaky_relu_fwd")
        self.inputs = x
        self.output = y
        return self.output

    def backward(self, dvalues):
        dy = to_device(dvalues)
        if self.fused_into_prev:
            self.dinputs = dy
            return self.dinputs
        dx = torch.empty_like(dy)
        check(lib().aether_leaky_relu_bwd(_ptr(self.inputs), _ptr(dy), _ptr(dx), dy.numel(), float(self._alpha),
                                          _stream()), "aether_leaky_relu_bwd")
        self.dinputs = dx
        return self.dinputs


class Leaky_ReLU(ReLU):
    """Drop-in for ``Leaky_ReLU`` (CNN_classes_cupy.py:417-428)."""

    def __init__(self, alpha=0.01):
        self.alpha = alpha

    @property
    def _alpha(self):
        return self.alpha


# ------------------------------------------------------------------------------------- dropout
class Layer_Dropout_Spatial(_Saved):
    """Drop-in for ``Layer_Dropout_Spatial`` (CNN_classes_cupy.py:384-404): one Bernoulli(keep) draw per
    channel, shared by the whole batch, scaled by 1/keep.  The draw uses NumPy's global generator like
    the reference's NumPy twin; ``channel_mask`` (1,1,1,C) may be overwritten before ``forward`` by
    setting ``fixed_mask``.  Output stays fp32 (the reference promotes to fp64 through its mask)."""

    _next_seed = 0xC4A7

    def __init__(self, rate):
        self.rate = rate
        self.keep_prob = 1 - rate
        self.fixed_mask = None
        self.seed = Layer_Dropout_Spatial._next_seed
        Layer_Dropout_Spatial._next_seed += 1
        self.step_dev = None            # int64 device counter: draw the mask on the device (CUDA-graph train step)
        self.fused_into_prev = False    # the Batch_Norm in front applies the mask (Model.finalize(fuse=True))

    def _restore_transient(self):
        self.fixed_mask = None
        self.step_dev = None
        self.fused_into_prev = False

    def draw_mask(self, Cc):
        """Draws this step's channel mask (Bernoulli(keep)/keep per channel) into ``channel_mask``."""
        if self.fixed_mask is None and self.step_dev is not None:
            self.channel_mask = _empty((1, 1, 1, Cc))
            check(lib().aether_channel_mask_dev(_ptr(self.channel_mask), Cc, float(self.keep_prob), self.seed,
                                                _ptr(self.step_dev), _stream()), "aether_channel_mask_dev")
        else:
            if self.fixed_mask is not None:
                mask = np.asarray(self.fixed_mask, dtype=np.float32).reshape(1, 1, 1, Cc)
            else:
                mask = (np.random.binomial(1, self.keep_prob, size=(1, 1, 1, Cc)) / self.keep_prob).astype(np.float32)
            self.channel_mask = to_device(mask)
        return self.channel_mask

    def forward(self, inputs, training):
        x = to_device(inputs)
        self.inputs = x
        if self.fused_into_prev:        # already masked by the fused Batch_Norm (training) / identity (inference)
            self.output = x
            return self.output
        if not training:
            self.output = x.clone()
            return self.output
        Cc = x.shape[-1]
        self.draw_mask(Cc)
        y = torch.empty_like(x)
        check(lib().aether_channel_scale(_ptr(x), _ptr(self.channel_mask), _ptr(y), x.numel(), Cc, _stream()),
              "aether_channel_scale")
        self.output = y
        return self.output

    def backward(self, dvalues):
        dy = to_device(dvalues)
        if self.fused_into_prev:
            self.dinputs = dy
            return self.dinputs
        dx = torch.empty_like(dy)
        check(lib().aether_channel_scale(_ptr(dy), _ptr(self.channel_mask), _ptr(dx), dy.numel(), dy.shape[-1],
                                         _stream()), "aether_channel_scale")
        self.dinputs = dx
        return self.dinputs


class Layer_Dropout(_Saved):
    """Drop-in for ``Layer_Dropout`` (CNN_classes_cupy.py:364-382).  ``rate`` is the drop rate; the
    element mask Bernoulli(1-rate)/(1-rate) is drawn on the device from a Philox stream keyed by
    ``seed`` and a per-call offset (``rank_offset`` separates data-parallel ranks)."""
    _next_seed = 0x5EED

    def __init__(self, rate, seed=None, rank_offset=0):
        self.rate = 1 - rate          # the reference stores the KEEP probability under this name (:367)
        if seed is None:
            seed = Layer_Dropout._next_seed
            Layer_Dropout._next_seed += 1
        self.seed = int(seed)
        self.rank_offset = int(rank_offset)
        self._calls = 0
        self.step_dev = None

    def _restore_transient(self):
        self.step_dev = None

    def forward(self, inputs, training):
        x = to_device(inputs)
        self.inputs = x
        if not training:
            self.output = x.clone()
            return self.output
        y = torch.empty_like(x)
        self.binary_mask = torch.empty_like(x)
        if self.step_dev is not None:   # the call counter lives on the device (CUDA-graph train step)
            check(lib().aether_dropout_fwd_dev(_ptr(x), _ptr(y), _ptr(self.binary_mask), x.numel(), float(self.rate),
                                               self.seed, self.rank_offset << 32, _ptr(self.step_dev), _stream()),
                  "aether_dropout_fwd_dev")
        else:
            offset = (self._calls << 40) + (self.rank_offset << 32)
            self._calls += 1
            check(lib().aether_dropout_fwd(_ptr(x), _ptr(y), _ptr(self.binary_mask), x.numel(), float(self.rate),
                                           self.seed, offset, _stream()), "aether_dropout_fwd")
        self.output = y
        return self.output

    def backward(self, dvalues):
        dy = to_device(dvalues)
        dx = torch.empty_like(dy)
        check(lib().aether_mul(_ptr(dy), _ptr(self.binary_mask), _ptr(dx), dy.numel(), _stream()), "aether_mul")
        self.dinputs = dx
        return self.dinputs


# ------------------------------------------------------------------------------------- Batch_Norm
class Batch_Norm(_Saved):
    """Drop-in for ``Batch_Norm`` (CNN_classes_cupy.py:430-526) for 4-D (NHWC) and 2-D inputs.
    ``gamma``/``beta`` (aliased as ``weights``/``biases``) have shape (C,); ``running_mean`` /
    ``running_var`` / ``batch_mean`` / ``batch_var`` are exposed with the reference's keep-dims shape
    ((1,1,1,C) or (1,C)) as views of flat (C,) storage.  ``normalized`` is not stored: the backward
    kernel recomputes x-hat from the saved statistics."""

    def __init__(self, epsilon=1e-5, momentum=0.9, n_features=None):
        self.epsilon = epsilon
        self.momentum = momentum
        self.gamma = None
        self.beta = None
        self.running_mean = None
        self.running_var = None
        self.weight_regularizer_l1 = 0
        self.weight_regularizer_l2 = 0
        self.bias_regularizer_l1 = 0
        self.bias_regularizer_l2 = 0
        self._ws = _Workspace()
        self._keep = None
        self.stats_from = None          # a Conv_Layer whose forward leaves `bn_partials` for this layer's input
        self.fused_alpha = None         # slope of the (Leaky_)ReLU applied inside this layer's kernels (None: not fused)
        self.fused_dropout = None       # a Layer_Dropout_Spatial behind that activation whose mask is applied here too
        self.fused_pool = None          # a max Pooling behind those whose windows are reduced here too
        self.pooled_now = False         # the last forward produced the pooled tensor
        self.lean = False               # do not write fp32 tensors whose only reader takes the bf16 copy (finalize(lean=True))
        self.copy_consumer = None       # the layer that reads the pooled tensor as x (its bf16 copy is written here)
        self.copy_dy_consumer = None    # the Conv_Layer in front (the bf16 copy of its dvalues is written here)
        if n_features is not None:
            self._create(n_features)

    def _restore_transient(self):
        self._ws = _Workspace()
        self._keep = None
        self.stats_from = None
        self.fused_alpha = None
        self.fused_dropout = None
        self.fused_pool = None
        self.pooled_now = False
        self.lean = False
        self.copy_consumer = None
        self.copy_dy_consumer = None
        if getattr(self, "gamma", None) is not None:
            self.running_mean = self._rm
            self.running_var = self._rv
        else:
            self.running_mean = self.running_var = None

    def _create(self, Cc):
        dev = _device()
        self.gamma = torch.ones(Cc, dtype=torch.float32, device=dev)
        self.beta = torch.zeros(Cc, dtype=torch.float32, device=dev)
        self._rm = torch.zeros(Cc, dtype=torch.float32, device=dev)
        self._rv = torch.ones(Cc, dtype=torch.float32, device=dev)
        self.running_mean = self._rm
        self.running_var = self._rv

    @property
    def weights(self):
        return self.gamma

    @weights.setter
    def weights(self, v):
        self.gamma = v

    @property
    def biases(self):
        return self.beta

    @biases.setter
    def biases(self, v):
        self.beta = v

    def forward(self, inputs, training):
        x = to_device(inputs)
        if x.ndim not in (2, 4):
            raise ValueError(f"Expected a 2D or 4D tensor, got {x.ndim} instead.")
        Cc = x.shape[-1]
        if self.gamma is None:
            self._create(Cc)
        rows = x.numel() // Cc
        keep = (1,) * (x.ndim - 1) + (Cc,)
        L = lib()
        ws = self._ws.get(L.aether_bn_workspace_bytes(rows, Cc))
        part = None
        if training:
            self._bm = _empty((Cc,))
            self._bv = _empty((Cc,))
            part = getattr(self.stats_from, "bn_partials", None) if self.stats_from is not None else None
            if part is not None and part[2] != x.data_ptr():
                part = None
        # Whole block tail in one pass: activation, dropout mask and a max pooling whose windows tile the input are
        # applied while x is read once; the activated tensor is never written (block_fused.cu).
        pool = self.fused_pool
        self.pooled_now = False
        if pool is not None and self.fused_alpha is not None and x.ndim == 4 and Cc % 4 == 0:
            fH, fW = pool.filter_size
            S, H, W = x.shape[0], x.shape[1], x.shape[2]
            if H % fH == 0 and W % fW == 0:
                mask = self.fused_dropout.draw_mask(Cc) if (training and self.fused_dropout is not None) else None
                pooled = _empty((S, H // fH, W // fW, Cc))
                self._pool_arg = _empty((S, H // fH, W // fW, Cc), torch.uint8)
                # the layer behind the pooling reads a bf16 copy of the pooled tensor: written by this same pass
                target = self.copy_consumer.x_copy_target(tuple(pooled.shape)) if self.copy_consumer is not None else None
                # x at every window's selected cell, for the backward statistics pass (training only)
                self._xsel = _empty(tuple(pooled.shape)) if training else None
                check(L.aether_bn_act_pool_fwd_copy(_ptr(x), _ptr(part[0]) if part else None, part[1] if part else 0,
                                                    _ptr(self.gamma), _ptr(self.beta), _ptr(self._rm), _ptr(self._rv),
                                                    _ptr(self._bm) if training else None, _ptr(self._bv) if training else None,
                                                    None if (self.lean and target) else _ptr(pooled), _ptr(self._pool_arg),
                                                    S, H, W, Cc, fH, fW,
                                                    float(self.epsilon), float(self.momentum), float(self.fused_alpha),
                                                    _ptr(mask), 1 if training else 0,
                                                    C.c_void_p(target[0]) if target else None, target[1] if target else 0,
                                                    _ptr(self._xsel), _ptr(ws), ws.numel(), _stream()),
                      "aether_bn_act_pool_fwd_copy")
                if target:
                    if self.lean:
                        _mark_unwritten(pooled)
                    self.copy_consumer.x_copy_written(pooled)
                self._fused_mask = mask
                self.pooled_now = True
                if training:
                    self.batch_mean = self._bm.view(keep)
                    self.batch_var = self._bv.view(keep)
                    self.running_mean = self._rm.view(keep)
                    self.running_var = self._rv.view(keep)
                self.inputs = x
                self.output = pooled
                return self.output
        y = torch.empty_like(x)
        if training:
            if self.fused_alpha is not None:
                # y = act(bn(x)) [* spatial-dropout mask] in the same passes; the layers behind only hand y through
                mask = self.fused_dropout.draw_mask(Cc) if self.fused_dropout is not None else None
                check(L.aether_bn_act_fwd_train(_ptr(x), _ptr(part[0]) if part else None, part[1] if part else 0,
                                                _ptr(self.gamma), _ptr(self.beta), _ptr(self._rm), _ptr(self._rv),
                                                _ptr(self._bm), _ptr(self._bv), _ptr(y), rows, Cc, float(self.epsilon),
                                                float(self.momentum), float(self.fused_alpha), _ptr(mask), _ptr(ws),
                                                ws.numel(), _stream()), "aether_bn_act_fwd_train")
                self._fused_mask = mask
            elif part is not None:
                # the convolution that produced x already reduced it per channel: merge its partials, read x once
                check(L.aether_bn_fwd_train_partials(_ptr(x), _ptr(part[0]), part[1], _ptr(self.gamma), _ptr(self.beta),
                                                     _ptr(self._rm), _ptr(self._rv), _ptr(self._bm), _ptr(self._bv),
                                                     _ptr(y), rows, Cc, float(self.epsilon), float(self.momentum),
                                                     _ptr(ws), ws.numel(), _stream()), "aether_bn_fwd_train_partials")
            else:
                check(L.aether_bn_fwd_train(_ptr(x), _ptr(self.gamma), _ptr(self.beta), _ptr(self._rm), _ptr(self._rv),
                                            _ptr(self._bm), _ptr(self._bv), _ptr(y), rows, Cc, float(self.epsilon),
                                            float(self.momentum), _ptr(ws), ws.numel(), _stream()), "aether_bn_fwd_train")
            self.batch_mean = self._bm.view(keep)
            self.batch_var = self._bv.view(keep)
            self.running_mean = self._rm.view(keep)       # the reference's stats pick up keep-dims here (:475-476)
            self.running_var = self._rv.view(keep)
        elif self.fused_alpha is not None:
            check(L.aether_bn_act_fwd_eval(_ptr(x), _ptr(self.gamma), _ptr(self.beta), _ptr(self._rm), _ptr(self._rv),
                                           _ptr(y), rows, Cc, float(self.epsilon), float(self.fused_alpha), _ptr(ws),
                                           ws.numel(), _stream()), "aether_bn_act_fwd_eval")
        else:
            check(L.aether_bn_fwd_eval(_ptr(x), _ptr(self.gamma), _ptr(self.beta), _ptr(self._rm), _ptr(self._rv),
                                       _ptr(y), rows, Cc, float(self.epsilon), _ptr(ws), ws.numel(), _stream()),
                  "aether_bn_fwd_eval")
        self.inputs = x
        self.output = y
        return self.output

    def backward(self, dvalues):
        dy = to_device(dvalues)
        x = self.inputs
        Cc = x.shape[-1]
        rows = x.numel() // Cc
        L = lib()
        ws = self._ws.get(L.aether_bn_workspace_bytes(rows, Cc))
        dx = torch.empty_like(x)
        if getattr(self, "_grad_views", None) is not None:
            self.dweights, self.dbiases = self._grad_views
        else:
            self.dweights = _empty((Cc,))
            self.dbiases = _empty((Cc,))
        if self.pooled_now:                  # dvalues is the gradient w.r.t. the POOLED output of the fused block tail
            S, H, W = x.shape[0], x.shape[1], x.shape[2]
            fH, fW = self.fused_pool.filter_size
            # dx is the dvalues of the convolution in front: its bf16 copy and the column sums for that layer's bias
            # gradient are written by this same pass
            conv = self.copy_dy_consumer
            target = conv.dy_copy_target() if (conv is not None and conv.output is x and 256 % max(Cc // 4, 1) == 0
                                               and Cc // 4 <= 256) else None
            rows = C.c_int(0)
            check(L.aether_bn_act_pool_bwd_copy(_ptr(x), _ptr(dy), _ptr(self._pool_arg), _ptr(self.gamma), _ptr(self.beta),
                                                _ptr(self._bm), _ptr(self._bv), None if (self.lean and target) else _ptr(dx),
                                                _ptr(self.dweights),
                                                _ptr(self.dbiases), S, H, W, Cc, fH, fW, float(self.epsilon),
                                                float(self.fused_alpha), _ptr(getattr(self, "_fused_mask", None)),
                                                C.c_void_p(target[0]) if target else None, target[1] if target else 0,
                                                C.c_void_p(target[2]) if target else None, target[3] if target else 0,
                                                C.byref(rows), _ptr(getattr(self, "_xsel", None)), _ptr(ws), ws.numel(),
                                                _stream()), "aether_bn_act_pool_bwd_copy")
            if target:
                if self.lean:
                    _mark_unwritten(dx)
                conv.dy_copy_written(dx, rows.value)
        elif self.fused_alpha is not None:   # dvalues is the gradient w.r.t. the ACTIVATED output
            check(L.aether_bn_act_bwd(_ptr(x), _ptr(self.beta), _ptr(dy), _ptr(self.gamma), _ptr(self._bm),
                                      _ptr(self._bv), _ptr(dx), _ptr(self.dweights), _ptr(self.dbiases), rows, Cc,
                                      float(self.epsilon), float(self.fused_alpha), _ptr(getattr(self, "_fused_mask", None)),
                                      _ptr(ws), ws.numel(), _stream()), "aether_bn_act_bwd")
        else:
            check(L.aether_bn_bwd(_ptr(x), _ptr(dy), _ptr(self.gamma), _ptr(self._bm), _ptr(self._bv), _ptr(dx),
                                  _ptr(self.dweights), _ptr(self.dbiases), rows, Cc, float(self.epsilon), _ptr(ws),
                                  ws.numel(), _stream()), "aether_bn_bwd")
        self.dinputs = dx
        return self.dinputs

    def get_parameters(self):
        return self.gamma, self.beta, self.running_mean, self.running_var

    def set_parameters(self, gamma, beta, running_mean, running_var):
        g = to_device(gamma).reshape(-1)
        if self.gamma is None:
            self._create(g.numel())
        self.gamma.copy_(g)
        self.beta.copy_(to_device(beta).reshape(-1))
        self._rm.copy_(to_device(running_mean).reshape(-1))
        self._rv.copy_(to_device(running_var).reshape(-1))


# ------------------------------------------------------------------------------------- Flatten / Dense
class Flatten(_Saved):
    """Drop-in for ``Flatten`` (CNN_classes_cupy.py:528-539); a view, no kernel."""

    def forward(self, inputs, training):
        x = to_device(inputs)
        self.inputs_shape = x.shape
        self.output = x.reshape(x.shape[0], -1)
        if getattr(x, "_aether_unwritten", False):
            _mark_unwritten(self.output)
        return self.output

    def backward(self, dvalues):
        self.dinputs = to_device(dvalues).reshape(self.inputs_shape)
        return self.dinputs


class Layer_Dense(_Saved):
    """Drop-in for ``Layer_Dense`` (CNN_classes_cupy.py:315-362).  The three products run through the
    convolution kernels as a 1x1 convolution on a 1x1 image (x (S,n_in) is NHWC with H=W=1; weights
    (n_in,n_out) are a (1,1,Cin,Cout) filter), so they use the same tensor-core path.  Parameters are
    fp32 (the reference's are fp64 because ``randn`` is); biases keep the (1, n_out) shape."""

    def __init__(self, n_inputs, n_neurons, weight_regularizer_l1=0, bias_regularizer_l1=0,
                 weight_regularizer_l2=0, bias_regularizer_l2=0, math_mode=None):
        w = 0.01 * np.random.randn(n_inputs, n_neurons) * np.sqrt(2.0 / n_inputs)       # :320-321
        self.weights = to_device(w.astype(np.float32))
        self.biases = torch.zeros((1, n_neurons), dtype=torch.float32, device=_device())
        self.weight_regularizer_l1 = weight_regularizer_l1
        self.weight_regularizer_l2 = weight_regularizer_l2
        self.bias_regularizer_l1 = bias_regularizer_l1
        self.bias_regularizer_l2 = bias_regularizer_l2
        self.math_mode = math_mode or DEFAULT_MATH_MODE
        self._ws = _Workspace()
        self._copies = _OperandCopies()
        self._handed = _HandedIn()

    def _restore_transient(self):
        self._ws = _Workspace()
        self._copies = _OperandCopies()
        self._handed = _HandedIn()

    def x_copy_target(self, shape):
        """(address, row length) where the bf16 copy of an input of `shape` (any shape that flattens to
        (samples, n_inputs), e.g. the pooled NHWC tensor in front of a Flatten) goes, or None."""
        n_in = self.weights.shape[0]
        total = 1
        for v in shape:
            total *= int(v)
        if len(shape) < 2 or total != int(shape[0]) * n_in:
            return None
        d = self._desc(int(shape[0]))
        lay = _operand_layout(d)
        # A row of the copy is one SAMPLE here, but the producer writes one PIXEL (shape[-1] channels) per row: the two
        # are the same bytes only when the sample's row is not padded (n_inputs a multiple of 64).
        if lay is None or lay.x_copy_ld != n_in:
            return None
        ws = self._ws.get(lib().aether_conv2d_workspace_bytes(C.byref(d)))
        return ws.data_ptr() + lay.x_copy_offset, int(shape[-1])

    def x_copy_written(self, x):
        self._handed.x = (self._ws.buf.data_ptr(), _array_tag(x))

    def _desc(self, S):
        n_in, n_out = self.weights.shape
        return AetherConvDesc(S, 1, 1, n_in, n_out, 1, 1, 1, 1, 0, 0, _lib.MATH_MODES[self.math_mode])

    def forward(self, inputs, training):
        x = to_device(inputs)
        if x.ndim != 2 or x.shape[1] != self.weights.shape[0]:
            raise ValueError(f"Layer_Dense expects (samples, {self.weights.shape[0]}), got {tuple(x.shape)}")
        d = self._desc(x.shape[0])
        L = lib()
        ws = self._ws.get(L.aether_conv2d_workspace_bytes(C.byref(d)))
        y = _empty((x.shape[0], self.weights.shape[1]))
        flags = _lib.CONV_X_COPY_READY if self._handed.x_ready(ws, x) else 0
        self._handed.x = None
        if not flags:
            _require_written(x, "Layer_Dense.forward")
        check(L.aether_conv2d_fwd_ex(C.byref(d), _ptr(x), _ptr(self.weights), _ptr(self.biases), _ptr(y), None, 0, _ptr(ws),
                                     ws.numel(), flags, _stream()), "aether_conv2d_fwd_ex")
        self.inputs = x
        self.output = y
        self._copies.record(ws, x, self.weights)
        return self.output

    def backward(self, dvalues):
        dy = to_device(dvalues)
        x = self.inputs
        d = self._desc(x.shape[0])
        L = lib()
        ws = self._ws.get(L.aether_conv2d_workspace_bytes(C.byref(d)))
        if getattr(self, "_grad_views", None) is not None:
            self.dweights, self.dbiases = self._grad_views
        else:
            self.dweights = torch.empty_like(self.weights)
            self.dbiases = torch.empty_like(self.biases)
        dx = torch.empty_like(x)
        copy_flags = self._copies.flags(ws, x, self.weights)
        if not (copy_flags & _lib.CONV_X_COPY_READY):
            _require_written(x, "Layer_Dense.backward")
        check(L.aether_conv2d_bwd(C.byref(d), _ptr(x), _ptr(dy), _ptr(self.weights), _ptr(dx), _ptr(self.dweights),
                                  _ptr(self.dbiases), _ptr(ws), ws.numel(), copy_flags, _stream()), "aether_conv2d_bwd")
        if self.weight_regularizer_l1 > 0 or self.weight_regularizer_l2 > 0:
            check(L.aether_regularizer_grad(_ptr(self.weights), _ptr(self.dweights), self.weights.numel(),
                                            float(self.weight_regularizer_l1), float(self.weight_regularizer_l2),
                                            _stream()), "aether_regularizer_grad")
        if self.bias_regularizer_l1 > 0 or self.bias_regularizer_l2 > 0:
            check(L.aether_regularizer_grad(_ptr(self.biases), _ptr(self.dbiases), self.biases.numel(),
                                            float(self.bias_regularizer_l1), float(self.bias_regularizer_l2),
                                            _stream()), "aether_regularizer_grad")
        self.dinputs = dx
        return self.dinputs

    def get_parameters(self):
        return self.weights, self.biases

    def set_parameters(self, weights, biases):
        self.weights.copy_(to_device(weights))
        self.biases.copy_(to_device(biases).reshape(1, -1))


# ------------------------------------------------------------------------------------- softmax / loss
def _labels_i32(y_true):
    """Targets as the kernels take them: class indices (int32, shape (rows,)) or, for 2-D input, the rows of target
    probabilities themselves (float32): one-hot or soft, the loss uses them as they are (CNN_classes_cupy.py:625-637)."""
    y = y_true if isinstance(y_true, torch.Tensor) else torch.as_tensor(np.asarray(y_true))
    if y.ndim == 2:
        return to_device(y, torch.float32)
    return to_device(y, torch.int32)


def _softmax_cce(z, labels, want_prob, want_loss, want_dz, want_correct, smooth_fwd, smooth_bwd, input_is_prob=False):
    rows, classes = z.shape
    prob = _empty((rows, classes)) if want_prob else None
    loss = _empty((rows,)) if want_loss else None
    dz = _empty((rows, classes)) if want_dz else None
    correct = _empty((rows,), torch.int32) if want_correct else None
    if labels is not None and labels.ndim == 2:
        if tuple(labels.shape) != (rows, classes):
            raise ValueError(f"targets have shape {tuple(labels.shape)}, expected {(rows, classes)}")
        check(lib().aether_softmax_cce_targets(_ptr(z), _ptr(labels), _ptr(prob), _ptr(loss), _ptr(dz), _ptr(correct), rows,
                                               classes, float(smooth_fwd), float(smooth_bwd), 1 if input_is_prob else 0,
                                               _stream()), "aether_softmax_cce_targets")
    else:
        check(lib().aether_softmax_cce(_ptr(z), _ptr(labels), _ptr(prob), _ptr(loss), _ptr(dz), _ptr(correct), rows,
                                       classes, float(smooth_fwd), float(smooth_bwd), 1 if input_is_prob else 0,
                                       _stream()), "aether_softmax_cce")
    return prob, loss, dz, correct


class SoftMax(_Saved):
    """Drop-in for ``SoftMax`` (CNN_classes_cupy.py:541-563).  ``backward`` is the reference's stand-alone Jacobian
    product (:549-560), as one kernel instead of a Python loop over the samples; networks that end in SoftMax +
    categorical cross-entropy take the combined backward (:666-680) and never call it."""

    def forward(self, inputs, training=True):
        z = to_device(inputs)
        self.inputs = z
        self.output, _, _, _ = _softmax_cce(z, None, True, False, False, False, 0.0, 0.0)
        return self.output

    def backward(self, dvalues):
        dv = to_device(dvalues)
        if tuple(dv.shape) != tuple(self.output.shape):
            raise ValueError(f"dvalues has shape {tuple(dv.shape)}, expected {tuple(self.output.shape)}")
        dx = torch.empty_like(dv)
        check(lib().aether_softmax_bwd(_ptr(self.output), _ptr(dv), _ptr(dx), dv.shape[0], dv.shape[1], _stream()),
              "aether_softmax_bwd")
        self.dinputs = dx
        return self.dinputs

    def predictions(self, outputs):
        return to_device(outputs).argmax(dim=1)


class Loss(_Saved):
    """Accumulating loss base class, ``Loss`` (CNN_classes_cupy.py:565-609)."""

    def remember_trainable_layers(self, trainable_layers):
        self.trainable_layers = trainable_layers

    def calculate(self, output, y, *, include_regularization=False, training=True):
        sample_losses = self.forward(output, y, training)
        data_loss = sample_losses.mean()
        self.accumulated_sum += sample_losses.sum()
        self.accumulated_count += len(sample_losses)
        if not include_regularization:
            return data_loss
        return data_loss, self.regularization_loss()

    def calculate_accumulated(self, *, include_regularization=False):
        data_loss = self.accumulated_sum / self.accumulated_count
        if not include_regularization:
            return data_loss
        return data_loss, self.regularization_loss()

    def new_pass(self):
        self.accumulated_sum = 0
        self.accumulated_count = 0

    def regularization_loss(self):
        out = None
        L = lib()
        for layer in self.trainable_layers:
            for arr, l1, l2 in ((layer.weights, layer.weight_regularizer_l1, layer.weight_regularizer_l2),
                                (layer.biases, layer.bias_regularizer_l1, layer.bias_regularizer_l2)):
                if l1 > 0 or l2 > 0:
                    if out is None:
                        out = torch.zeros(1, dtype=torch.float32, device=_device())
                    check(L.aether_regularizer_loss(_ptr(arr), arr.numel(), float(l1), float(l2), _ptr(out),
                                                    _stream()), "aether_regularizer_loss")
        return out[0] if out is not None else 0


class Loss_CategoricalCrossEntropy(Loss):
    """Drop-in for ``Loss_CategoricalCrossEntropy`` (CNN_classes_cupy.py:611-652); ``y_pred`` are
    probabilities, ``y_true`` class indices or one-hot rows."""

    def __init__(self, label_smoothing=0.0):
        self.label_smoothing = label_smoothing

    def forward(self, y_pred, y_true, training=True):
        p = to_device(y_pred)
        smooth = self.label_smoothing if training else 0.0
        _, loss, _, _ = _softmax_cce(p, _labels_i32(y_true), False, True, False, False, smooth, 0.0, input_is_prob=True)
        return loss

    def backward(self, dvalues, y_true):
        p = to_device(dvalues)
        _, _, dz, _ = _softmax_cce(p, _labels_i32(y_true), False, False, True, False, 0.0, self.label_smoothing,
                                   input_is_prob=True)
        self.dinputs = dz
        return self.dinputs


class Activation_Softmax_Loss_CategoricalCrossEntropy:
    """Drop-in for the combined class (CNN_classes_cupy.py:654-680); ``backward`` takes the softmax
    OUTPUT and returns (p - y_smooth)/samples."""

    def __init__(self, label_smoothing=0.0):
        self.activation = SoftMax()
        self.loss = Loss_CategoricalCrossEntropy(label_smoothing)
        self.label_smoothing = label_smoothing

    def forward(self, inputs, y_true, training=True):
        self.activation.forward(inputs, training)
        self.output = self.activation.output
        return self.loss.calculate(self.output, y_true, training=training)

    def backward(self, dvalues, y_true, training=True):
        p = to_device(dvalues)
        smooth = self.label_smoothing if training else 0.0
        _, _, dz, _ = _softmax_cce(p, _labels_i32(y_true), False, False, True, False, 0.0, smooth, input_is_prob=True)
        self.dinputs = dz
        return self.dinputs


# ------------------------------------------------------------------------------------- Adam
class Optimizer_Adam(_Saved):
    """Drop-in for ``Optimizer_Adam`` (CNN_classes_cupy.py:685-736).  State lives on the layer under the
    reference's attribute names (``weight_momentums``, ``weight_cache``, ``bias_momentums``,
    ``bias_cache``) and parameters are updated in place.  ``grad_scale`` multiplies every gradient
    first (1/world_size turns an all-reduced sum into the data-parallel average)."""

    def __init__(self, learning_rate=.001, decay=0., epsilon=1e-7, beta_1=0.9, beta_2=.999):
        self.learning_rate = learning_rate
        self.current_learning_rate = learning_rate
        self.decay = decay
        self.iterations = 0
        self.epsilon = epsilon
        self.beta_1 = beta_1
        self.beta_2 = beta_2
        self.grad_scale = 1.0
        self.step_dev = None            # int64 device copy of `iterations` (CUDA-graph train step)

    def _restore_transient(self):
        self.step_dev = None

    def pre_update_parameters(self):
        if self.decay:
            self.current_learning_rate = self.learning_rate * (1. / (1. + self.decay * self.iterations))

    def _step(self, p, g, m, v):
        if self.step_dev is not None:   # iterations, decay and bias corrections evaluated on the device
            check(lib().aether_adam_step_dev(_ptr(p), _ptr(g), _ptr(m), _ptr(v), p.numel(), float(self.learning_rate),
                                             float(self.decay), float(self.beta_1), float(self.beta_2),
                                             float(self.epsilon), float(self.grad_scale), _ptr(self.step_dev),
                                             _stream()), "aether_adam_step_dev")
            return
        t = self.iterations + 1
        check(lib().aether_adam_step(_ptr(p), _ptr(g), _ptr(m), _ptr(v), p.numel(), float(self.current_learning_rate),
                                     float(self.beta_1), float(self.beta_2), float(self.epsilon),
                                     float(1 - self.beta_1 ** t), float(1 - self.beta_2 ** t), float(self.grad_scale),
                                     _stream()), "aether_adam_step")

    def update_parameters(self, layer):
        if not hasattr(layer, "weight_cache"):
            layer.weight_momentums = torch.zeros_like(layer.weights)
            layer.weight_cache = torch.zeros_like(layer.weights)
            layer.bias_momentums = torch.zeros_like(layer.biases)
            layer.bias_cache = torch.zeros_like(layer.biases)
        self._step(layer.weights, layer.dweights, layer.weight_momentums, layer.weight_cache)
        self._step(layer.biases, layer.dbiases, layer.bias_momentums, layer.bias_cache)

    def update_flat(self, params, grads, m, v):
        """One launch over a flat parameter buffer (used by the data-parallel trainer)."""
        self._step(params, grads, m, v)

    def post_update_parameters(self):
        self.iterations += 1
