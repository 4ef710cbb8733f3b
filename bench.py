#!/usr/bin/env python
"""Benchmark of the convolution hot path: Conv_Layer forward + backward (dX, dW, dB).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--mode bf16|tf32]

Workload (default): the largest shape of the isolated conv sweep -- batch 256 per GPU, NHWC
56x56, 64 -> 128 channels, 3x3, stride 1, 'same', x ~ N(0,1), He-normal filters, dy ~ N(0,1),
synthetic and seeded.  One step = one forward + one backward of the layer; with N > 1 every rank
works on its own batch shard (weak scaling) and the flat dW/dB buffer is all-reduced over NCCL.
FLOP count per step and GPU: 6 * S*Ho*Wo * 9*Cin*Cout (forward + dX + dW as dense GEMMs).

Prints ONE JSON line (rank 0).  `value` = whole-job TFLOP/s with inputs resident in HBM, `e2e` =
the same through the layer API from pinned host buffers (host<->device copies timed), `roofline` =
the dominant kernel against the measured tensor peak, `cpu_baseline` = the NumPy restatement of the
reference path on the host cores (a bounded sample).  `--impl reference` times only that CPU path.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPE = dict(S=256, H=56, W=56, Cin=64, Cout=128, f=3)
WORKLOAD = "conv_fwd_bwd S=256 NHWC 56x56 Cin=64 Cout=128 3x3 stride1 same (largest shape of the isolated sweep)"
CPU_SAMPLE_IMAGES = 24       # images of the same shape per CPU-baseline sample
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the three GEMM kernels on this workload (bf16, batch 256),
# from the one-pass ncu capture summarised in profiles/conv_fwd_bwd_56x56_64to128_dram_traffic.txt.  Part of each
# kernel's output is still dirty in L2 when it ends, so the written bytes are below the algorithmic 411 / 205 MB.
DRAM_TRAFFIC_S256 = {"igemm_fwd": 102975744 + 353941760, "igemm_dx": 205719808 + 155275776, "dw": 308393216 + 356096}
REF_STEP_IMAGES = 2          # images per step of the --impl reference arm


def conv_flops(S, H, W, Cin, Cout, f):
    return 6.0 * S * H * W * f * f * Cin * Cout


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return dict(burst=p["bf16_tflops"], sustained=p["bf16_tflops_sustained"], hbm=p["hbm_gbs"], source="measured")
    return dict(burst=1590.0, sustained=1400.0, hbm=6650.0, source="fallback")


# ----------------------------------------------------------------------------------- CPU arm
def cpu_threads():
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    return max(1, min(n, 64))


def cpu_conv_sample(images, threads=1, min_seconds=0.0, max_passes=1):
    """Times the oracle's einsum formulation (the reference's own algorithm: strided windows + np.einsum in
    float32, whose C loops are single-threaded) on `images` images of the benchmark shape.  The reference itself
    never uses more than one core; to give the CPU every core of the box the batch is split over `threads` worker
    threads, each running the same code on its images (einsum releases the GIL).  The pass over the sample is
    repeated until `min_seconds` of CPU work have been timed (at most `max_passes` passes).
    Returns (TFLOP/s, seconds, passes)."""
    from concurrent.futures import ThreadPoolExecutor
    from oracle import aether_oracle as O
    rng = np.random.default_rng(4)
    s = SHAPE
    x = rng.standard_normal((images, s["H"], s["W"], s["Cin"])).astype(np.float32)
    w = (rng.standard_normal((s["f"], s["f"], s["Cin"], s["Cout"])) * np.sqrt(2.0 / (9 * s["Cin"]))).astype(np.float32)
    b = np.zeros(s["Cout"], np.float32)
    dy = rng.standard_normal((images, s["H"], s["W"], s["Cout"])).astype(np.float32)
    threads = max(1, min(threads, images))
    bounds = [(images * k // threads, images * (k + 1) // threads) for k in range(threads)]

    def work(lohi):
        lo, hi = lohi
        y = O.conv_forward(x[lo:hi], w, b, dtype=np.float32)
        dx, dw, db = O.conv_backward(x[lo:hi], w, dy[lo:hi], dtype=np.float32)
        return dw, db

    t0 = time.perf_counter()
    passes = 0
    while True:
        if threads == 1:
            parts = [work(bounds[0])]
        else:
            with ThreadPoolExecutor(threads) as ex:
                parts = list(ex.map(work, bounds))
        dw = sum(p[0] for p in parts)                  # the per-chunk filter gradients add up to the batch's
        passes += 1
        dt = time.perf_counter() - t0
        if dt >= min_seconds or passes >= max_passes:
            break
    fl = passes * conv_flops(images, s["H"], s["W"], s["Cin"], s["Cout"], s["f"])
    return fl / dt / 1e12, dt, passes


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    s = SHAPE
    threads = cpu_threads()
    images = max(REF_STEP_IMAGES, threads)
    for _ in range(args.warmup):
        cpu_conv_sample(images, threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_conv_sample(images, threads)
    dt = time.perf_counter() - t0
    fl = conv_flops(images, s["H"], s["W"], s["Cin"], s["Cout"], s["f"]) * args.steps
    val = fl / dt / 1e12
    sample = ("%d images of the workload shape per step, NumPy einsum over strided windows in float32 (the reference's "
              "algorithm) on %d worker threads" % (images, threads))
    print(json.dumps({
        "impl": "reference", "metric": "conv_fwd_bwd_tflops", "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ----------------------------------------------------------------------------------- clocks
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows = []
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [c.strip() for c in line.split(",")]))

    def stop(self, t_begin, t_end):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [r for t, r in self.rows if t_begin <= t <= t_end + 0.2 and len(r) >= 7] or [r for _, r in self.rows if len(r) >= 7]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = sorted(float(r[0]) for r in rows)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for k, n in enumerate(names) if any(r[3 + k].lower().startswith("active") for r in rows)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": float(rows[0][1]), "reasons": reasons, "samples": len(rows),
                "power_w_max": max(float(r[2]) for r in rows)}


# ----------------------------------------------------------------------------------- GPU arm
def run_gpu(args):
    import ctypes as C
    import torch
    import torch.distributed as dist
    from aether_ml_b200 import _lib
    from aether_ml_b200.layers import Conv_Layer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    L = _lib.lib()
    s = SHAPE
    S, H, W, Cin, Cout, f = s["S"], s["H"], s["W"], s["Cin"], s["Cout"], s["f"]

    np.random.seed(1234)                                  # identical filters on every rank
    layer = Conv_Layer((H, W, Cin), Cout, (f, f), (1, 1), "same", math_mode=args.mode)
    g = torch.Generator(device="cpu").manual_seed(100 + rank)
    x_host = torch.randn((S, H, W, Cin), generator=g, dtype=torch.float32).pin_memory()
    dy_host = torch.randn((S, H, W, Cout), generator=g, dtype=torch.float32).pin_memory()
    x = x_host.to(dev)
    dy = dy_host.to(dev)
    flat = torch.zeros(layer.filter_weights.numel() + Cout, dtype=torch.float32, device=dev)
    layer._grad_views = (flat[:layer.filter_weights.numel()].view(layer.filter_weights.shape), flat[-Cout:])

    def step():
        layer.forward(x, True)
        layer.backward(dy)
        if world > 1:
            dist.all_reduce(flat)

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    sync_all()
    if _lib.device_status() != 0:
        raise RuntimeError("a kernel abandoned a bounded wait: status %d" % _lib.device_status())

    # ---- timed region: device-resident inputs
    sampler = ClockSampler(local) if rank == 0 else None
    # Per-kernel CUDA events on every n-th launch of each kind, n >= 5 (an odd stride, so the two alternating cast
    # launches are both sampled): an event pair costs a few microseconds of stream time, ~6 % of this step when taken everywhere.
    prof_stride = max(5, (args.steps // 8) | 1) if args.steps >= 10 else 1      # about eight samples per kind, odd
    L.aether_profile_enable(prof_stride)
    launches0 = _lib.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    t_begin = time.perf_counter()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    sync_all()
    t_end = time.perf_counter()
    launches = _lib.launch_count() - launches0
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_total = float(ms.item())
    kinds = {}
    for kind, name in enumerate(["igemm_fwd", "igemm_dx", "dw", "operand_cast"]):
        tot, n = C.c_double(0), C.c_int(0)
        L.aether_profile_read(kind, C.byref(tot), C.byref(n))
        kinds[name] = (tot.value, n.value)
    L.aether_profile_enable(0)
    clocks = sampler.stop(t_begin, t_end) if sampler else None

    # ---- end to end: pinned host buffers in, results back to the host, every step
    y_out = torch.empty((S, H, W, Cout), dtype=torch.float32).pin_memory()
    dx_out = torch.empty((S, H, W, Cin), dtype=torch.float32).pin_memory()
    g_out = torch.empty(flat.numel(), dtype=torch.float32).pin_memory()

    # Three streams, two sets of device input buffers: the upload of step k+1 and the download of step k run
    # in both directions of the PCIe link at once, the layer runs on the launching stream in between.  Every
    # step still uploads its own inputs and downloads its own y, dX, dW/dB.
    s_main = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    xd = [torch.empty_like(x) for _ in range(2)]
    dyd = [torch.empty_like(dy) for _ in range(2)]
    ev_in = [torch.cuda.Event() for _ in range(2)]      # inputs of this buffer set are on the device
    ev_free = [torch.cuda.Event() for _ in range(2)]    # the layer has finished reading this buffer set
    ev_comp, ev_out = torch.cuda.Event(), torch.cuda.Event()
    e2e_count = [0]

    def e2e_step():
        k = e2e_count[0] & 1
        first = e2e_count[0] < 2
        e2e_count[0] += 1
        with torch.cuda.stream(s_in):
            if not first:
                s_in.wait_event(ev_free[k])
            xd[k].copy_(x_host, non_blocking=True)
            dyd[k].copy_(dy_host, non_blocking=True)
            ev_in[k].record(s_in)
        s_main.wait_event(ev_in[k])
        if e2e_count[0] > 1:
            s_main.wait_event(ev_out)                   # the layer's output buffers are reused: previous download first
        y = layer.forward(xd[k], True)
        dxd = layer.backward(dyd[k])
        if world > 1:
            dist.all_reduce(flat)
        ev_free[k].record(s_main)
        ev_comp.record(s_main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_comp)
            y_out.copy_(y, non_blocking=True)
            dx_out.copy_(dxd, non_blocking=True)
            g_out.copy_(flat, non_blocking=True)
            ev_out.record(s_out)

    e2e_steps = max(4, min(args.steps, 10))
    e2e_step()
    sync_all()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(e2e_steps):
        e2e_step()
    s_main.wait_event(ev_out)                           # the last download is inside the timed region
    f1.record()
    sync_all()
    ms2 = torch.tensor([f0.elapsed_time(f1)], device=dev)
    if world > 1:
        dist.all_reduce(ms2, op=dist.ReduceOp.MAX)
    e2e_ms = float(ms2.item()) / e2e_steps

    if rank == 0:
        pk = peaks()
        fl_step = conv_flops(S, H, W, Cin, Cout, f)
        ms_step = ms_total / args.steps
        value = fl_step * world / (ms_step * 1e-3) / 1e12
        per_gemm = fl_step / 3.0
        dom = max(("igemm_fwd", "igemm_dx", "dw"), key=lambda k: kinds[k][0])
        dom_ms = kinds[dom][0] / max(kinds[dom][1], 1)
        achieved = per_gemm / (dom_ms * 1e-3) / 1e12 if dom_ms > 0 else None
        peak = pk["sustained"] if ms_total > 1500 else pk["burst"]
        cpu_thr = cpu_threads()
        cpu_imgs = max(CPU_SAMPLE_IMAGES, 4 * cpu_thr)
        cpu_val, cpu_s, cpu_passes = (None, 0.0, 0) if args.skip_cpu_baseline else cpu_conv_sample(cpu_imgs, cpu_thr, 10.0, 64)
        out = {
            "metric": "conv_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": args.mode, "data": "synthetic",
            "config": {"workload": WORKLOAD if S == 256 else WORKLOAD.replace("S=256", "S=%d" % S), "per_gpu_batch": S, "flops_per_step_per_gpu": fl_step,
                       "l2": "inputs (x 205 MB, dy 411 MB per step) exceed the 126 MB L2; no explicit flush",
                       "parallelism": "dp%d batch-sharded, one NCCL all-reduce of dW/dB per step" % world if world > 1 else "single GPU",
                       "pct_of_bf16_peak_burst": 100.0 * value / world / pk["burst"],
                       "pct_of_bf16_peak_sustained": 100.0 * value / world / pk["sustained"]},
            "e2e": {"value": fl_step * world / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": (x_host.numel() + dy_host.numel()) * 4,
                    "d2h_bytes_per_step": (y_out.numel() + dx_out.numel() + g_out.numel()) * 4},
            "gpu_launches": int(launches),
            "roofline": {"bound": "tensor", "kernel": dom, "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": (achieved / peak) if achieved else None,
                         "traffic": DRAM_TRAFFIC_S256.get(dom) if (S == 256 and args.mode == "bf16") else None,
                         "traffic_unit": "bytes per launch (dram read + write, ncu, full-size workload)",
                         "peak_source": "%s (%s bf16 figure of MEASURED_PEAKS.json)" % (pk["source"], "sustained" if ms_total > 1500 else "burst"),
                         "launch_ms": dom_ms, "flops_per_launch": per_gemm,
                         "timed_launches": kinds[dom][1], "timed_every": prof_stride},
            "kernels": {k: {"total_ms": v[0], "launches": v[1], "avg_ms": v[0] / max(v[1], 1),
                            "tflops": (per_gemm / (v[0] / max(v[1], 1) * 1e-3) / 1e12) if (v[1] and k != "operand_cast" and v[0] > 0) else None}
                        for k, v in kinds.items()},
            "cpu_baseline": {"value": cpu_val, "unit": "TFLOP/s", "cores": cpu_thr, "kind": "port",
                             "sample": "%d images of the workload shape, fwd+bwd %d times (%.1f s), NumPy einsum over strided windows in float32 as in the reference, batch split over %d worker threads" % (cpu_imgs, cpu_passes, cpu_s, cpu_thr)},
            "clocks": clocks,
        }
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


# ----------------------------------------------------------------------------------- training workload
def build_cnn(widen, math_mode, fuse=False):
    """The CIFAR-shaped 3-block CNN of the reference's README example (CNN/architectures/CNN_cifar1.py:16-55):
    Conv 3->32->64->128 (3x3 same) each with Batch_Norm / ReLU / [spatial dropout] / 2x2 max pool, Dense
    2048->256 LeakyReLU dropout, Dense 256->10, softmax + CCE (label smoothing 0.01), Adam lr 1e-3 decay 5e-5.
    `widen`=4 gives the data-parallel configuration (channels 128/256/512, Dense 8192->1024->10)."""
    from aether_ml_b200 import layers as Ly
    from aether_ml_b200.model import Accuracy_Categorical, Model
    m = Model()
    c_in, hw = 3, 32
    for k, (c_out, sd) in enumerate(((32 * widen, 0.075), (64 * widen, 0.1), (128 * widen, None))):
        m.add(Ly.Conv_Layer((hw, hw, c_in), c_out, (3, 3), (1, 1), "same", math_mode=math_mode))
        m.add(Ly.Batch_Norm(n_features=c_out))
        m.add(Ly.ReLU())
        if sd:
            m.add(Ly.Layer_Dropout_Spatial(sd))
        m.add(Ly.Pooling((2, 2), (2, 2), "valid", "max"))
        c_in, hw = c_out, hw // 2
    m.add(Ly.Flatten())
    m.add(Ly.Layer_Dense(4 * 4 * c_in, 256 * widen, weight_regularizer_l2=2e-5, math_mode=math_mode))
    m.add(Ly.Leaky_ReLU(0.01))
    m.add(Ly.Layer_Dropout(0.075, seed=11))
    m.add(Ly.Layer_Dense(256 * widen, 10, math_mode=math_mode))
    m.add(Ly.SoftMax())
    m.set(loss=Ly.Loss_CategoricalCrossEntropy(label_smoothing=0.01),
          optimizer=Ly.Optimizer_Adam(learning_rate=1e-3, decay=5e-5), accuracy=Accuracy_Categorical())
    m.finalize(flat=True, fuse=fuse)
    return m


def run_train(args):
    """Training images/s of the 3-block CNN, batch-sharded over the ranks (global batch fixed: strong scaling);
    one step = forward + loss gradient + backward + all-reduce of the flat gradient buffer + Adam."""
    import torch
    import torch.distributed as dist
    from aether_ml_b200 import _lib, dp
    world, rank, local = dp.init_from_env()
    dev = torch.device("cuda", local)
    widen = 4 if args.workload == "train_wide" else 1
    global_batch = args.global_batch or (4096 if widen == 4 else 128)
    lo, hi = dp.shard_bounds(global_batch, rank, world)
    np.random.seed(7)                                   # same initial parameters on every rank
    model = build_cnn(widen, args.mode, args.fuse)
    dp.attach(model)
    g = torch.Generator(device="cpu").manual_seed(3)
    X_host = torch.rand((global_batch, 32, 32, 3), generator=g)[lo:hi].contiguous().pin_memory()
    y_host = torch.randint(0, 10, (global_batch,), generator=g, dtype=torch.int32)[lo:hi].contiguous().pin_memory()
    X, y = X_host.to(dev), y_host.to(dev)

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    l0 = _lib.launch_count()
    for _ in range(max(args.warmup, 3)):
        model.train_step(X, y)
    sync_all()
    launches_per_step = (_lib.launch_count() - l0) // max(args.warmup, 3)
    if _lib.device_status() != 0:
        raise RuntimeError("a kernel abandoned a bounded wait: status %d" % _lib.device_status())
    step = model.train_step
    if args.graph:                                      # the whole step (all-reduce included) as one CUDA-graph launch
        model.capture_train_step(X, y)
        step = model.train_step_graph
        for _ in range(3):
            step(X, y)
        sync_all()
    sampler = ClockSampler(local) if rank == 0 else None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    t_begin = time.perf_counter()
    e0.record()
    for _ in range(args.steps):
        step(X, y)
    e1.record()
    sync_all()
    t_end = time.perf_counter()
    launches = launches_per_step * args.steps           # kernels of this library executed (replayed when --graph)
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_step = float(ms.item()) / args.steps
    clocks = sampler.stop(t_begin, t_end) if sampler else None

    def e2e_step():
        out = step(X_host.to(dev, non_blocking=True), y_host.to(dev, non_blocking=True))
        return out[:1].cpu()                             # read part of the step's result back every step

    e2e_step()
    sync_all()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n_e2e = max(2, min(args.steps, 10))
    f0.record()
    for _ in range(n_e2e):
        e2e_step()
    f1.record()
    sync_all()
    ms2 = torch.tensor([f0.elapsed_time(f1)], device=dev)
    if world > 1:
        dist.all_reduce(ms2, op=dist.ReduceOp.MAX)
    e2e_ms = float(ms2.item()) / n_e2e
    if rank == 0:
        print(json.dumps({
            "metric": "train_images_per_s", "value": global_batch / (ms_step * 1e-3), "unit": "images/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": args.mode, "data": "synthetic",
            "config": {"workload": "train step of the CIFAR-shaped 3-block CNN%s, global batch %d NHWC (32,32,3) ~ U[0,1), "
                                   "Adam lr 1e-3 decay 5e-5" % (" widened 4x (128/256/512, Dense 8192->1024->10)" if widen == 4 else "", global_batch),
                       "per_gpu_batch": hi - lo, "parallelism": "dp%d, one NCCL all-reduce of the flat gradient buffer per step" % world,
                       "l2": "activations of a step (GBs) exceed the 126 MB L2", "params": int(model.flat_params.numel()),
                       "cuda_graph": bool(args.graph), "fused_bn_relu": bool(args.fuse)},
            "e2e": {"value": global_batch / (e2e_ms * 1e-3), "unit": "images/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": (X_host.numel() * 4 + y_host.numel() * 4) * world, "d2h_bytes_per_step": 40 * world},
            "gpu_launches": int(launches), "clocks": clocks}))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="conv", choices=["conv", "train", "train_wide"],
                    help="conv = isolated Conv_Layer fwd+bwd (default, the headline metric); train / train_wide = "
                         "training images/s of the 3-block CNN (README size / widened 4x, global batch 4096)")
    ap.add_argument("--global-batch", type=int, default=0)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--mode", default="bf16", choices=["bf16", "tf32"])
    ap.add_argument("--batch", type=int, default=SHAPE["S"], help="per-GPU batch (smaller only for profiler captures)")
    ap.add_argument("--skip-cpu-baseline", action="store_true", help="omit the CPU sample (profiler captures)")
    ap.add_argument("--graph", action="store_true", help="train workloads: replay the step from a captured CUDA graph")
    ap.add_argument("--fuse", action="store_true",
                    help="train workloads: apply each ReLU inside the Batch_Norm kernels in front of it (finalize(fuse=True))")
    args = ap.parse_args()
    SHAPE["S"] = args.batch
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "conv":
        run_gpu(args)
    else:
        run_train(args)


if __name__ == "__main__":
    main()
