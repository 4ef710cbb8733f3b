"""``Model`` orchestration with the public surface of Aether-ML's ``CNN/models/CNN_model_cupy.py``
(add / set / finalize / train / forward / backward / evaluate / predict / get_parameters /
set_parameters / save_parameters / load_parameters), driving the device layers of
:mod:`aether_ml_b200.layers`.  It holds no arithmetic: layers are duck-typed exactly as in the
reference (``forward(inputs, training)`` sets ``.output``, ``backward(dvalues)`` sets ``.dinputs``;
a layer is trainable when it has a ``weights`` attribute, CNN_model_cupy.py:52-53).

Additions that the reference does not have, all optional:
  * ``finalize(flat=True)`` packs every trainable layer's parameters and gradients into two flat
    device buffers (views keep the per-layer attribute names), so one Adam launch and -- under data
    parallelism -- one all-reduce cover the whole network;
  * ``train_step(X, y)`` runs one forward/backward/update without printing or host synchronisation.
"""
import pickle

import numpy as np
import torch

from .layers import (Activation_Softmax_Loss_CategoricalCrossEntropy, Batch_Norm, Conv_Layer, Layer_Dropout_Spatial,
                     Loss_CategoricalCrossEntropy, Pooling, ReLU, SoftMax, to_device, _labels_i32)


class Layer_Input:
    """Feeds the batch to the first layer (CNN_model_cupy.py:389-391)."""

    def forward(self, inputs, training):
        self.output = inputs


class Accuracy:
    """Running accuracy (CNN_model_cupy.py:344-363)."""

    def calculate(self, predictions, y):
        hits = self.compare(predictions, y)
        self.accumulated_sum += hits.sum()
        self.accumulated_count += len(hits)
        return hits.float().mean()

    def calculate_accumulated(self):
        return self.accumulated_sum / self.accumulated_count

    def new_pass(self):
        self.accumulated_sum = 0
        self.accumulated_count = 0


class Accuracy_Categorical(Accuracy):
    """CNN_model_cupy.py:380-387: exact match of class indices (one-hot targets are arg-maxed)."""

    def init(self, y):
        pass

    def compare(self, predictions, y):
        y = y if isinstance(y, torch.Tensor) else torch.as_tensor(np.asarray(y))
        y = y.to(predictions.device)
        if y.ndim == 2:
            y = y.argmax(dim=1)
        return predictions == y


class Accuracy_Regression(Accuracy):
    """CNN_model_cupy.py:367-378: |prediction - y| below std(y)/250."""

    def __init__(self):
        self.precision = None

    def init(self, y, reinit=False):
        if self.precision is None or reinit:
            self.precision = float(np.std(np.asarray(y.cpu() if isinstance(y, torch.Tensor) else y))) / 250

    def compare(self, predictions, y):
        y = to_device(y)
        return (predictions - y).abs() < self.precision


def _batches(n, batch_size):
    if batch_size is None:
        return [slice(None)]
    steps = -(-n // batch_size)
    return [slice(k * batch_size, (k + 1) * batch_size) for k in range(steps)]


class Model:
    def __init__(self):
        self.layers = []
        self.softmax_classifier_output = None
        self.loss = None
        self.optimizer = None
        self.accuracy = None
        self.flat_params = None
        self.grad_hook = None      # callable(flat_grads) run between backward and the optimizer (all-reduce)

    def add(self, layer):
        self.layers.append(layer)

    def set(self, *, loss=None, optimizer=None, accuracy=None):
        if loss is not None:
            self.loss = loss
        if optimizer is not None:
            self.optimizer = optimizer
        if accuracy is not None:
            self.accuracy = accuracy

    # ------------------------------------------------------------------ wiring
    def finalize(self, flat=False, fuse=False):
        self.input_layer = Layer_Input()
        chain = [self.input_layer] + self.layers + [self.loss]
        for pos, layer in enumerate(self.layers, start=1):
            layer.prev = chain[pos - 1]
            layer.next = chain[pos + 1]
        self.output_layer_activation = self.layers[-1]
        # A Batch_Norm directly behind a Conv_Layer takes its batch statistics from the convolution's epilogue
        # (when the kernel that serves the shape provides them) instead of reducing the activation again.
        for a, b in zip(self.layers[:-1], self.layers[1:]):
            if isinstance(a, Conv_Layer) and isinstance(b, Batch_Norm):
                a.emit_bn_stats = True
                b.stats_from = a
            # fuse=True: a ReLU / Leaky_ReLU directly behind a Batch_Norm is applied by the Batch_Norm's own kernels
            # (one read and one write of the activation less each way).  The Batch_Norm's `output` is then the
            # ACTIVATED tensor and the activation layer hands its input through unchanged.
            if fuse and isinstance(a, Batch_Norm) and isinstance(b, ReLU):
                a.fused_alpha = float(b._alpha)
                b.fused_into_prev = True
                # ... and a Layer_Dropout_Spatial behind that activation: its per-channel mask is folded into the
                # Batch_Norm's per-channel coefficients (act(v) * m = act(m * v) for m >= 0)
                c = getattr(b, "next", None)
                if isinstance(c, Layer_Dropout_Spatial):
                    a.fused_dropout = c
                    c.fused_into_prev = True
                    c = getattr(c, "next", None)
                # ... and a max Pooling with stride == filter behind those: the Batch_Norm then reads the convolution
                # output once and writes the pooled tensor; the activated tensor in between is never materialised
                # (decided per call: the windows must tile the input)
                if (isinstance(c, Pooling) and c.pooling_type == "max" and c.padding == "valid"
                        and tuple(c.strides) == tuple(c.filter_size)):
                    a.fused_pool = c
                    c.fused_bn = a
        self.trainable_layers = [l for l in self.layers if hasattr(l, "weights")]
        if self.loss is not None:
            self.loss.remember_trainable_layers(self.trainable_layers)
        if isinstance(self.layers[-1], SoftMax) and isinstance(self.loss, Loss_CategoricalCrossEntropy):
            self.softmax_classifier_output = Activation_Softmax_Loss_CategoricalCrossEntropy(self.loss.label_smoothing)
        if flat:
            self._pack_flat()

    def _pack_flat(self):
        """Move all parameters into one flat buffer and pre-allocate one flat gradient buffer plus
        Adam state; the layers keep seeing arrays of their usual shapes (views)."""
        pending = [l for l in self.trainable_layers if l.weights is None]
        if pending:
            raise RuntimeError("finalize(flat=True) needs every trainable layer to own its parameters already "
                               "(give Batch_Norm n_features)")
        sizes = []
        for l in self.trainable_layers:
            sizes += [l.weights.numel(), l.biases.numel()]
        # keep every view 16-byte aligned
        offs, total = [], 0
        for n in sizes:
            offs.append(total)
            total += (n + 3) // 4 * 4
        dev = self.trainable_layers[0].weights.device
        self.flat_params = torch.zeros(total, dtype=torch.float32, device=dev)
        self.flat_grads = torch.zeros(total, dtype=torch.float32, device=dev)
        self.flat_m = torch.zeros(total, dtype=torch.float32, device=dev)
        self.flat_v = torch.zeros(total, dtype=torch.float32, device=dev)
        k = 0
        for l in self.trainable_layers:
            views = []
            for name in ("weights", "biases"):
                old = getattr(l, name)
                o, n = offs[k], sizes[k]
                k += 1
                pv = self.flat_params[o:o + n].view(old.shape)
                pv.copy_(old)
                setattr(l, name, pv)
                views.append(self.flat_grads[o:o + n].view(old.shape))
                mom = "weight" if name == "weights" else "bias"
                setattr(l, mom + "_momentums", self.flat_m[o:o + n].view(old.shape))
                setattr(l, mom + "_cache", self.flat_v[o:o + n].view(old.shape))
            l._grad_views = tuple(views)

    # ------------------------------------------------------------------ passes
    def forward(self, X, training):
        self.input_layer.forward(X, training)
        for layer in self.layers:
            layer.forward(layer.prev.output, training)
        return layer.output

    def backward(self, output, y):
        if self.softmax_classifier_output is not None:
            self.softmax_classifier_output.backward(output, y, training=True)
            self.layers[-1].dinputs = self.softmax_classifier_output.dinputs
            upstream = self.layers[:-1]
        else:
            self.loss.backward(output, y)
            upstream = self.layers
        first = self.layers[0]
        for layer in reversed(upstream):
            if layer is first and hasattr(layer, "_desc"):
                layer.backward(layer.next.dinputs, need_dinputs=False)   # nobody consumes d(loss)/d(images)
            else:
                layer.backward(layer.next.dinputs)

    def _apply_optimizer(self, run_hook=True):
        opt = self.optimizer
        if run_hook and self.grad_hook is not None and self.flat_params is not None:
            self.grad_hook(self.flat_grads)
        opt.pre_update_parameters()
        if self.flat_params is not None and hasattr(opt, "update_flat"):
            opt.update_flat(self.flat_params, self.flat_grads, self.flat_m, self.flat_v)
        else:
            for layer in self.trainable_layers:
                opt.update_parameters(layer)
        opt.post_update_parameters()
        if getattr(self, "_g_step", None) is not None:
            self._g_step.add_(1)            # device copy of the step count (see enable_device_step)

    def train_step(self, X, y):
        """forward + loss gradient + backward + optimizer for one batch; returns the logits' softmax."""
        output = self.forward(X, training=True)
        self.backward(output, y)
        self._apply_optimizer()
        return output

    # ------------------------------------------------------------------ CUDA-graph train step
    def enable_device_step(self):
        """Moves the per-step host state (Adam's iteration count, the dropout call counters) into one int64 device
        counter that every train step increments; the channel masks of spatial dropout are then drawn on the device.
        Required for a captured train step, usable on its own (same numbers eagerly and replayed)."""
        if getattr(self, "_g_step", None) is None:
            dev = self.trainable_layers[0].weights.device
            self._g_step = torch.full((1,), int(self.optimizer.iterations), dtype=torch.int64, device=dev)
            for obj in [self.optimizer] + [l for l in self.layers if hasattr(l, "step_dev")]:
                obj.step_dev = self._g_step
        return self._g_step

    def _graph_body(self):
        return self.train_step(self._g_X, self._g_y)

    def _graph_state(self):
        """Every tensor a train step changes besides activations: parameters, Adam moments, running statistics."""
        ts = [self.flat_params, self.flat_m, self.flat_v, self._g_step]
        for l in self.layers:
            if isinstance(l, Batch_Norm) and l.gamma is not None:
                ts += [l._rm, l._rv]
        return ts

    def capture_train_step(self, X, y, warmup=2):
        """Records ``train_step`` for batches shaped like (X, y) into a CUDA graph; ``train_step_graph`` replays
        it with one launch (two, around the gradient hook, when one is set).  A step of the small reference
        networks is ~130 kernel launches of a few microseconds
        each, so the eager step is bound by launch overhead, not by the GPU.  Needs ``finalize(flat=True)``.
        Whatever the reference changes on the host per step (Adam's iteration count and decayed learning rate,
        the dropout draws) is read from one int64 device counter that the graph itself increments.  The warm-up
        steps (they size the workspaces) are undone, so capturing does not train."""
        if self.flat_params is None:
            raise RuntimeError("capture_train_step needs finalize(flat=True)")
        self._g_X = to_device(X).clone()
        self._g_y = _labels_i32(y).clone()
        opt = self.optimizer
        self.enable_device_step()
        saved = [t.clone() for t in self._graph_state()]
        saved_it = opt.iterations
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(max(int(warmup), 1)):
                self._graph_body()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        for t, s in zip(self._graph_state(), saved):
            t.copy_(s)
        # With a gradient hook (the data-parallel all-reduce) the step is recorded as two graphs and the hook runs
        # eagerly between them: collectives stay outside stream capture, where a rank that fails cannot leave
        # its peers waiting inside a captured collective.
        self._graph = torch.cuda.CUDAGraph()
        self._graph_opt = None
        with torch.cuda.graph(self._graph):
            self._g_out = self.forward(self._g_X, training=True)
            self.backward(self._g_out, self._g_y)
            if self.grad_hook is None:
                self._apply_optimizer()
        if self.grad_hook is not None:
            self._graph_opt = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self._graph_opt):
                self._apply_optimizer(run_hook=False)
        opt.iterations = saved_it           # capture records work, it does not run it
        return self._graph

    def train_step_graph(self, X, y):
        """One training step by replaying the captured graph on a new batch of the captured shape."""
        if getattr(self, "_graph", None) is None:
            raise RuntimeError("train_step_graph called before capture_train_step")
        self._g_X.copy_(to_device(X), non_blocking=True)
        self._g_y.copy_(_labels_i32(y), non_blocking=True)
        self._graph.replay()
        if self._graph_opt is not None:
            self.grad_hook(self.flat_grads)
            self._graph_opt.replay()
        opt = self.optimizer
        opt.pre_update_parameters()         # host mirror of what the graph just did on the device
        opt.post_update_parameters()
        return self._g_out

    def train(self, X, y, *, epochs=1, batch_size=None, print_every=1, validation_data=None):
        self.accuracy.init(y)
        chunks = _batches(len(X), batch_size)
        print("Training")
        for epoch in range(1, epochs + 1):
            print(f' epoch: {epoch}')
            self.loss.new_pass()
            self.accuracy.new_pass()
            for step, sl in enumerate(chunks):
                batch_X, batch_y = X[sl], y[sl]
                output = self.forward(batch_X, training=True)
                data_loss, regularization_loss = self.loss.calculate(output, batch_y, include_regularization=True,
                                                                     training=True)
                loss = data_loss + regularization_loss
                predictions = self.output_layer_activation.predictions(output)
                accuracy = self.accuracy.calculate(predictions, batch_y)
                self.backward(output, batch_y)
                self._apply_optimizer()
                if not step % print_every or step == len(chunks) - 1:
                    print(f'epoch: {epoch}, acc: {float(accuracy):.3f}, loss: {float(loss):.3f} ('
                          f'data_loss: {float(data_loss):.3f}, reg_loss: {float(regularization_loss):.3f}, '
                          f'lr:: {self.optimizer.current_learning_rate}')
        epoch_data_loss, epoch_regularization_loss = self.loss.calculate_accumulated(include_regularization=True)
        epoch_loss = epoch_data_loss + epoch_regularization_loss
        epoch_accuracy = self.accuracy.calculate_accumulated()
        print(f' training, acc: {float(epoch_accuracy):.3f}, loss: {float(epoch_loss):.3f} ('
              f'data_loss: {float(epoch_data_loss):.3f}, reg_loss: {float(epoch_regularization_loss):.3f}, '
              f'lr:: {self.optimizer.current_learning_rate}')
        if validation_data is not None:
            self.evaluate(*validation_data, batch_size=batch_size)

    def evaluate(self, X_val, y_val, *, batch_size=None):
        self.loss.new_pass()
        self.accuracy.new_pass()
        for sl in _batches(len(X_val), batch_size):
            output = self.forward(X_val[sl], training=False)
            self.loss.calculate(output, y_val[sl], training=False)
            self.accuracy.calculate(self.output_layer_activation.predictions(output), y_val[sl])
        validation_loss = self.loss.calculate_accumulated()
        validation_accuracy = self.accuracy.calculate_accumulated()
        print(f'Valdiation, acc: {float(validation_accuracy):.3f}, loss: {float(validation_loss):.3f}')
        return float(validation_accuracy), float(validation_loss)

    def predict(self, X, *, batch_size=None):
        outs = [self.forward(X[sl], training=False).clone() for sl in _batches(len(X), batch_size)]
        return torch.vstack(outs)

    # ------------------------------------------------------------------ parameters
    def get_parameters(self):
        return [layer.get_parameters() for layer in self.trainable_layers]

    def set_parameters(self, parameters):
        for parameter_set, layer in zip(parameters, self.trainable_layers):
            layer.set_parameters(*parameter_set)

    def save_parameters(self, path):
        """Same on-disk format as the reference (a pickled list of per-layer tuples,
        CNN_model_cupy.py:277-282), with NumPy arrays so the file loads without a GPU."""
        host = [tuple(np.asarray(a.detach().cpu()) for a in params) for params in self.get_parameters()]
        with open(path, 'wb') as f:
            pickle.dump(host, f)

    def load_parameters(self, path):
        with open(path, 'rb') as f:
            self.set_parameters(pickle.load(f))

    load_paramters = load_parameters      # spelling used by the reference's NumPy model and two of its scripts
