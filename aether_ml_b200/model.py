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

from .layers import (Activation_Softmax_Loss_CategoricalCrossEntropy, Batch_Norm, Conv_Layer, Flatten, Layer_Dropout_Spatial,
                     Loss_CategoricalCrossEntropy, Pooling, ReLU, SoftMax, to_device, _labels_i32, _softmax_cce, _Saved)


class Layer_Input:
    """Feeds the batch to the first layer (CNN_model_cupy.py:389-391)."""

    def forward(self, inputs, training):
        self.output = inputs


class Accuracy(_Saved):
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
        self._graph = self._graph_opt = None
        self._graph_metrics = False
        self._m_last = self._m_sum = None
        self.bucket_reducer = None # dp.BucketReducer: all-reduces the flat gradients bucket by bucket during backward
        self._bucket_of_layer = {}
        self._update_stream = None # side stream on which finished buckets are updated while backward goes on
        self._updated_early = set()

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
    # ------------------------------------------------------------------ whole-model files
    def __getstate__(self):
        """What ``save`` writes: the layer list, loss, optimizer and accuracy objects (each without its per-step
        arrays) and the options of the last ``finalize``; flat buffers, graphs and wiring are rebuilt on loading."""
        return {"layers": self.layers, "loss": self.loss, "optimizer": self.optimizer, "accuracy": self.accuracy,
                "finalize_options": getattr(self, "_finalize_options", None)}

    def __setstate__(self, state):
        self.__init__()
        self.layers = state["layers"]
        self.loss, self.optimizer, self.accuracy = state["loss"], state["optimizer"], state["accuracy"]
        if state.get("finalize_options") is not None:
            had_state = [(l, {n: getattr(l, n) for n in ("weight_momentums", "weight_cache", "bias_momentums", "bias_cache")
                              if hasattr(l, n)}) for l in self.layers]
            self.finalize(**state["finalize_options"])
            for l, st in had_state:                      # Adam's moments go back into the (possibly flat) state arrays
                for n, arr in st.items():
                    if getattr(l, n) is not arr:
                        getattr(l, n).copy_(arr.reshape(getattr(l, n).shape))

    def save(self, path):
        """Writes the whole model to one file (``Model.save``, CNN_model_cupy.py:291-309).  As in the reference the
        per-step arrays (inputs, outputs, gradients) and the accumulated loss / accuracy are left out; parameters,
        Adam's state, running statistics and the layer configuration are kept.  Device arrays are stored as NumPy
        arrays; the file is a pickle of this package's classes (it is not interchangeable with the reference's own
        whole-model pickles, which name the reference's modules)."""
        if self.loss is not None:
            self.loss.new_pass()
        if self.accuracy is not None:
            self.accuracy.new_pass()
        with open(path, 'wb') as f:
            pickle.dump(self, f)

    @staticmethod
    def load(path):
        """Reads a file written by ``save`` (``Model.load``, CNN_model_cupy.py:311-317) and returns the model, wired
        with the same ``finalize`` options it had and ready to predict or to go on training."""
        with open(path, 'rb') as f:
            model = pickle.load(f)
        if not isinstance(model, Model):
            raise TypeError("%s does not hold a Model" % path)
        return model

    def finalize(self, flat=False, fuse=False, lean=False):
        """Wires the layers (CNN_model_cupy.py:27-64).  Beyond the reference: `flat` packs parameters and gradients
        into flat buffers, `fuse` merges each block tail into one pass each way, and `lean` (with `fuse`) stops
        writing fp32 tensors that only this library's own next kernel would read and that kernel reads as a bf16
        operand copy anyway: the pooled output of a fused block tail in front of a Conv_Layer / Dense, and the dx of a
        fused tail behind a tensor-core Conv_Layer.  Parameters, gradients and outputs of the model are the same
        numbers as without it; the `.output` of such a Pooling and the `.dinputs` of such a Batch_Norm are then
        placeholders (a layer asked to read one raises)."""
        self._finalize_options = {"flat": bool(flat), "fuse": bool(fuse), "lean": bool(lean)}
        self.input_layer = Layer_Input()
        chain = [self.input_layer] + self.layers + [self.loss]
        for pos, layer in enumerate(self.layers, start=1):
            layer.prev = chain[pos - 1]
            layer.next = chain[pos + 1]
        self.output_layer_activation = self.layers[-1]
        if isinstance(self.layers[0], Conv_Layer):
            self.layers[0].first_in_model = True        # backward never asks it for dinputs
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
                    # The pooled tensor is the x of the layer behind (through a Flatten, if any) and the dx of this
                    # block tail is the dvalues of the convolution in front: the tail's kernels write the bf16 copies
                    # those layers' tensor-core kernels read, so neither runs a cast pass over the fp32 tensor.
                    nxt = getattr(c, "next", None)
                    if isinstance(nxt, Flatten):
                        nxt = getattr(nxt, "next", None)
                    if hasattr(nxt, "x_copy_target"):
                        a.copy_consumer = nxt
                    a.lean = bool(lean)
                    if isinstance(getattr(a, "prev", None), Conv_Layer):
                        a.copy_dy_consumer = a.prev
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
        # element range of each trainable layer (its weights, biases and padding), in forward order: contiguous
        bounds = offs[0::2] + [total]
        self.flat_layer_ranges = [(bounds[i], bounds[i + 1]) for i in range(len(self.trainable_layers))]
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

    def set_bucket_reducer(self, reducer):
        """Installs a gradient reducer (see dp.BucketReducer): bucket i is started as soon as the backward pass has
        written the gradients of its last layer, and waited for right before that bucket's optimizer update."""
        self.bucket_reducer = reducer
        self._bucket_of_layer = {}
        if reducer is not None:
            for i, (_, _, trigger) in enumerate(reducer.buckets):
                self._bucket_of_layer[id(self.trainable_layers[trigger])] = i

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
            b = self._bucket_of_layer.get(id(layer))
            if b is not None:                   # this layer's gradients complete a bucket: start reducing it
                self.bucket_reducer.start(b)
                self._update_bucket_early(b)

    def _update_bucket_early(self, b):
        """Every bucket but the last is updated as soon as its all-reduce is through, on a side stream, while the
        main stream goes on back-propagating the layers in front: nobody reads those parameters again in this step
        (their layers' backward is over), and the update -- Adam moves 28 bytes per parameter, the dense head is most
        of them -- runs beside tensor-bound convolution kernels instead of after them."""
        r = self.bucket_reducer
        if b == len(r.buckets) - 1 or self.flat_params is None or not hasattr(self.optimizer, "update_flat"):
            return
        if self._update_stream is None:
            self._update_stream = torch.cuda.Stream()
        main = torch.cuda.current_stream()
        side = self._update_stream
        side.wait_stream(main)
        self.optimizer.pre_update_parameters()          # this step's learning rate (idempotent within a step)
        lo, hi, _ = r.buckets[b]
        with torch.cuda.stream(side):
            r.wait(b)
            self.optimizer.update_flat(self.flat_params[lo:hi], self.flat_grads[lo:hi], self.flat_m[lo:hi], self.flat_v[lo:hi])
        self._updated_early.add(b)

    def _apply_optimizer(self, run_hook=True):
        opt = self.optimizer
        if run_hook and self.grad_hook is not None and self.flat_params is not None:
            self.grad_hook(self.flat_grads)
        opt.pre_update_parameters()
        if self.bucket_reducer is not None and self.flat_params is not None and hasattr(opt, "update_flat"):
            # one update per bucket, each behind its own all-reduce only (the first bucket's update overlaps the
            # second bucket's all-reduce)
            if self._updated_early:
                torch.cuda.current_stream().wait_stream(self._update_stream)
            for i, (lo, hi, _) in enumerate(self.bucket_reducer.buckets):
                if i in self._updated_early:
                    continue
                if run_hook:
                    self.bucket_reducer.wait(i)
                opt.update_flat(self.flat_params[lo:hi], self.flat_grads[lo:hi], self.flat_m[lo:hi], self.flat_v[lo:hi])
            self._updated_early = set()
        elif self.flat_params is not None and hasattr(opt, "update_flat"):
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
        out = self.train_step(self._g_X, self._g_y)
        if self._graph_metrics:
            self._step_metrics(out, self._g_y)
        return out

    def _step_metrics(self, output, labels):
        """This step's data loss, accuracy and regularisation loss, kept on the device: `_m_last` holds the three
        values of the latest step, `_m_sum` the running sums of the per-sample losses and of the hits that the
        reference accumulates on the host (CNN_model_cupy.py:104-111, CNN_classes_cupy.py:577-589)."""
        smooth = self.loss.label_smoothing
        _, rows_loss, _, hits = _softmax_cce(output, labels, False, True, False, True, smooth, 0.0, input_is_prob=True)
        self._m_last[0:1].copy_(rows_loss.mean().reshape(1))
        self._m_last[1:2].copy_(hits.float().mean().reshape(1))
        reg = self.loss.regularization_loss()
        if isinstance(reg, torch.Tensor):
            self._m_last[2:3].copy_(reg.reshape(1))
        else:
            self._m_last[2:3].fill_(float(reg))
        self._m_sum[0] += rows_loss.sum()
        self._m_sum[1] += hits.sum()

    def _graph_state(self):
        """Every tensor a train step changes besides activations: parameters, Adam moments, running statistics."""
        ts = [self.flat_params, self.flat_m, self.flat_v, self._g_step, self._m_last, self._m_sum]
        for l in self.layers:
            if isinstance(l, Batch_Norm) and l.gamma is not None:
                ts += [l._rm, l._rv]
        return ts

    def _all_ranks_agree(self, ok):
        """True when `ok` holds on every rank (one small eager all-reduce; single process: `ok` itself)."""
        import torch.distributed as dist
        if not (dist.is_initialized() and dist.get_world_size() > 1):
            return ok
        flag = torch.tensor([1.0 if ok else 0.0], device=self.flat_params.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        return bool(flag.item() > 0.5)

    def capture_train_step(self, X, y, warmup=2, collectives_in_graph=True, metrics=False):
        """Records ``train_step`` for batches shaped like (X, y) into a CUDA graph; ``train_step_graph`` replays
        it with one launch.  A step of the small reference networks is ~130 kernel launches of a few microseconds
        each, so the eager step is bound by launch overhead, not by the GPU.  Needs ``finalize(flat=True)``.
        Whatever the reference changes on the host per step (Adam's iteration count and decayed learning rate,
        the dropout draws) is read from one int64 device counter that the graph itself increments.  The warm-up
        steps (they size the workspaces) are undone, so capturing does not train.

        Data parallelism: the bucketed all-reduces (dp.BucketReducer) are recorded inside the same graph, forked
        onto NCCL's stream where the backward pass starts them and joined before each bucket's update.  The
        capture runs in thread-local error mode: the process group's watchdog thread polls CUDA events of earlier
        collectives, which a global-mode capture treats as an illegal call and aborts with -- on that rank only.
        A rank whose capture failed must not leave its peers inside a recorded collective, so after the attempt
        every rank reports over one eager all-reduce and, unless all succeeded, all fall back to two graphs with
        the collectives launched eagerly between them.  ``collectives_in_graph=False`` asks for that form.
        ``metrics=True`` also records the step's loss / accuracy bookkeeping (``Model.train`` uses it)."""
        if self.flat_params is None:
            raise RuntimeError("capture_train_step needs finalize(flat=True)")
        self._g_X = to_device(X).clone()
        self._g_y = _labels_i32(y).clone()
        opt = self.optimizer
        dev = self.flat_params.device
        self.enable_device_step()
        self._graph_metrics = bool(metrics)
        if getattr(self, "_m_last", None) is None:
            self._m_last = torch.zeros(3, dtype=torch.float32, device=dev)
            self._m_sum = torch.zeros(2, dtype=torch.float64, device=dev)
        saved = [t.clone() for t in self._graph_state()]
        saved_it = opt.iterations
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(max(int(warmup), 1)):
                self._graph_body()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        for t, sv in zip(self._graph_state(), saved):
            t.copy_(sv)
        reducer = self.bucket_reducer if (self.bucket_reducer is not None and self.bucket_reducer.active) else None
        eager_between = self.grad_hook is not None or (reducer is not None and not collectives_in_graph)
        self._graph = self._graph_opt = None
        self.capture_note = "one graph"
        if reducer is not None and not eager_between:
            graph, ok, err = torch.cuda.CUDAGraph(), True, ""
            outer = torch.cuda.current_stream()
            try:
                with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                    self._g_out = self._graph_body()
            except Exception as e:                  # noqa: BLE001 -- any failure means "do not replay this graph"
                ok, err = False, repr(e)
                reducer.works = [None] * len(reducer.buckets)
                torch.cuda.set_stream(outer)        # a failed capture may leave its side stream current
            if self._all_ranks_agree(ok):
                self._graph = graph
                self.capture_note = "one graph with %d all-reduce bucket(s) inside" % len(reducer.buckets)
            else:
                eager_between = True
                self.capture_note = "two graphs, collectives eager (in-graph capture failed on a rank%s)" % (": " + err if err else "")
        if self._graph is None:
            # With collectives outside: graph 1 = forward + backward (no bucket is started inside it), then the
            # reduction runs eagerly, then graph 2 = the optimizer.
            self._graph = torch.cuda.CUDAGraph()
            held, self._bucket_of_layer = self._bucket_of_layer, {}
            try:
                with torch.cuda.graph(self._graph, capture_error_mode="thread_local"):
                    self._g_out = self.forward(self._g_X, training=True)
                    self.backward(self._g_out, self._g_y)
                    if not eager_between:
                        self._apply_optimizer()
                        if self._graph_metrics:
                            self._step_metrics(self._g_out, self._g_y)
            finally:
                self._bucket_of_layer = held
            if eager_between:
                self._graph_opt = torch.cuda.CUDAGraph()
                with torch.cuda.graph(self._graph_opt, capture_error_mode="thread_local"):
                    self._apply_optimizer(run_hook=False)
                    if self._graph_metrics:
                        self._step_metrics(self._g_out, self._g_y)
                if self.capture_note == "one graph":
                    self.capture_note = "two graphs, collectives eager"
        opt.iterations = saved_it           # capture records work, it does not run it
        return self._graph

    def release_graphs(self):
        """Drops the captured graphs (and the batch buffers they read).  A graph that recorded collectives keeps the
        NCCL communicator busy for as long as it exists: destroying the process group while such a graph is alive
        waits for ever, so data-parallel programs call this (or ``dp.shutdown``) before tearing the group down."""
        self._graph = self._graph_opt = None
        self._g_out = None
        self._graph_metrics = False
        if torch.cuda.is_available():
            torch.cuda.synchronize()

    def train_step_graph(self, X, y):
        """One training step by replaying the captured graph on a new batch of the captured shape."""
        if getattr(self, "_graph", None) is None:
            raise RuntimeError("train_step_graph called before capture_train_step")
        self._g_X.copy_(to_device(X), non_blocking=True)
        self._g_y.copy_(_labels_i32(y), non_blocking=True)
        self._graph.replay()
        if self._graph_opt is not None:
            if self.grad_hook is not None:
                self.grad_hook(self.flat_grads)
            elif self.bucket_reducer is not None:
                self.bucket_reducer.reduce_all()
            self._graph_opt.replay()
        opt = self.optimizer
        opt.pre_update_parameters()         # host mirror of what the graph just did on the device
        opt.post_update_parameters()
        return self._g_out

    def _graph_train_possible(self, X, y, chunks):
        """The captured step serves ``train`` when every batch has the same shape and the step is the combined
        softmax + cross-entropy one on flat parameters."""
        if self.flat_params is None or self.softmax_classifier_output is None or not torch.cuda.is_available():
            return False
        if not isinstance(self.accuracy, Accuracy_Categorical) or len(chunks) == 0:
            return False
        sizes = {len(range(*sl.indices(len(X)))) for sl in chunks}
        return len(sizes) == 1

    def train(self, X, y, *, epochs=1, batch_size=None, print_every=1, validation_data=None, use_graph=None):
        """The reference's training loop (CNN_model_cupy.py:67-151), same printed lines.  When every batch has the
        same shape and the model was finalized with ``flat=True`` the step is captured once and replayed
        (``use_graph=None`` decides by itself, True / False force it): loss and accuracy are then computed and
        accumulated on the device inside the replayed step and read back only for the lines that are printed,
        so the loop never waits for the GPU in between."""
        self.accuracy.init(y)
        chunks = _batches(len(X), batch_size)
        graph = self._graph_train_possible(X, y, chunks) if use_graph is None else bool(use_graph)
        if graph and not self._graph_train_possible(X, y, chunks):
            raise RuntimeError("use_graph=True needs finalize(flat=True), softmax + categorical cross-entropy, "
                               "Accuracy_Categorical and batches of one size")
        print("Training")
        if graph:
            first = chunks[0]
            shape = tuple(to_device(X[first]).shape)
            if getattr(self, "_graph", None) is None or not self._graph_metrics or tuple(self._g_X.shape) != shape:
                self.capture_train_step(X[first], y[first], metrics=True)
            per_batch = shape[0]
        for epoch in range(1, epochs + 1):
            print(f' epoch: {epoch}')
            self.loss.new_pass()
            self.accuracy.new_pass()
            if graph:
                self._m_sum.zero_()
            for step, sl in enumerate(chunks):
                batch_X, batch_y = X[sl], y[sl]
                if graph:
                    self.train_step_graph(batch_X, batch_y)
                    data_loss, accuracy, regularization_loss = self._m_last[0], self._m_last[1], self._m_last[2]
                    loss = None
                else:
                    output = self.forward(batch_X, training=True)
                    data_loss, regularization_loss = self.loss.calculate(output, batch_y, include_regularization=True,
                                                                         training=True)
                    loss = data_loss + regularization_loss
                    predictions = self.output_layer_activation.predictions(output)
                    accuracy = self.accuracy.calculate(predictions, batch_y)
                    self.backward(output, batch_y)
                    self._apply_optimizer()
                if not step % print_every or step == len(chunks) - 1:
                    if graph:                   # one read-back of the three device scalars, only for printed steps
                        data_loss, accuracy, regularization_loss = (float(v) for v in self._m_last.tolist())
                        loss = data_loss + regularization_loss
                    print(f'epoch: {epoch}, acc: {float(accuracy):.3f}, loss: {float(loss):.3f} ('
                          f'data_loss: {float(data_loss):.3f}, reg_loss: {float(regularization_loss):.3f}, '
                          f'lr:: {self.optimizer.current_learning_rate}')
            if graph:                           # hand the device-side sums to the reference's accumulators
                self.loss.accumulated_sum = self._m_sum[0].float()
                self.loss.accumulated_count = per_batch * len(chunks)
                self.accuracy.accumulated_sum = self._m_sum[1].float()
                self.accuracy.accumulated_count = per_batch * len(chunks)
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

    def save_parameters(self, path, include_optimizer=False):
        """Same on-disk format as the reference (a pickled list of per-layer tuples,
        CNN_model_cupy.py:277-282), with NumPy arrays so the file loads without a GPU.
        ``include_optimizer=True`` (not in the reference, whose checkpoints drop Adam's state) writes a dict
        {"parameters": that list, "optimizer": iteration count + per-layer moment arrays} instead, so training
        resumes with the same moments and decayed learning rate."""
        host = [tuple(np.asarray(a.detach().cpu()) for a in params) for params in self.get_parameters()]
        payload = host
        if include_optimizer:
            state = []
            for l in self.trainable_layers:
                if hasattr(l, "weight_cache"):
                    state.append(tuple(np.asarray(getattr(l, n).detach().cpu()) for n in
                                       ("weight_momentums", "weight_cache", "bias_momentums", "bias_cache")))
                else:
                    state.append(None)
            payload = {"parameters": host,
                       "optimizer": {"iterations": int(self.optimizer.iterations), "layers": state}}
        with open(path, 'wb') as f:
            pickle.dump(payload, f)

    def load_parameters(self, path):
        """Reads a checkpoint written by ``save_parameters`` here or by the reference (CNN_model_cupy.py:284-289).
        The reference's CuPy model pickles ``cupy`` arrays; they are rebuilt as NumPy arrays (the pickle stores
        them as host arrays wrapped in a ``cupy._core.core.array`` call), so such files load without CuPy.  Only
        array reconstruction is allowed while unpickling; anything else in the file is refused."""
        with open(path, 'rb') as f:
            payload = _CheckpointUnpickler(f).load()
        if isinstance(payload, dict):
            self.set_parameters(payload["parameters"])
            opt_state = payload.get("optimizer")
            if opt_state is not None and self.optimizer is not None:
                self.optimizer.iterations = int(opt_state["iterations"])
                self.optimizer.pre_update_parameters()
                step_dev = getattr(self, "_g_step", None)
                if step_dev is not None:
                    step_dev.fill_(self.optimizer.iterations)
                for l, st in zip(self.trainable_layers, opt_state["layers"]):
                    if st is None:
                        continue
                    for name, arr in zip(("weight_momentums", "weight_cache", "bias_momentums", "bias_cache"), st):
                        cur = getattr(l, name, None)
                        t = to_device(arr)
                        if cur is not None:
                            cur.copy_(t.reshape(cur.shape))     # in place: flat-buffer views stay views
                        else:
                            setattr(l, name, t.clone())
        else:
            self.set_parameters(payload)

    load_paramters = load_parameters      # spelling used by the reference's NumPy model and two of its scripts


class _CheckpointUnpickler(pickle.Unpickler):
    """Unpickler for parameter checkpoints: NumPy's array reconstruction helpers, and ``cupy`` array
    constructors mapped to ``numpy.asarray``; every other global is refused."""

    _NUMPY = {("numpy._core.multiarray", "_reconstruct"), ("numpy.core.multiarray", "_reconstruct"),
              ("numpy._core.multiarray", "scalar"), ("numpy.core.multiarray", "scalar"),
              ("numpy", "ndarray"), ("numpy", "dtype")}

    def find_class(self, module, name):
        if module.split(".")[0] == "cupy" and name in ("array", "asarray", "ndarray"):
            if name == "ndarray":
                raise pickle.UnpicklingError("cupy.ndarray subclass state is not a parameter checkpoint")
            return np.asarray
        if (module, name) in self._NUMPY:
            return super().find_class(module, name)
        raise pickle.UnpicklingError("checkpoint refers to %s.%s, which is not an array constructor" % (module, name))
