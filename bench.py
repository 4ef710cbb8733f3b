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
the kernel kind that takes the largest share of the step against its measured peak (tensor or HBM),
`cpu_baseline` = the reference path on the host cores (a bounded sample).  The same line carries
`train` = training images/s of the widened 3-block CNN at global batch 4096 sharded over the N
ranks (strong scaling; fused block tails, one captured graph per step, bucketed all-reduce),
`dp_check` (N > 1) = the bucket-reduced gradient buffer against an all-gathered sum, and at N = 1
`sweep` = the four shapes of the isolated conv sweep in bf16 and TF32 plus the first config.
`--impl reference` times only the CPU path.
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
# dram__bytes_read.sum + dram__bytes_write.sum per launch on this workload (bf16, batch 256), from the one-pass ncu
# capture of one step summarised in profiles/conv_step_56x56_64to128_dram_traffic.txt.  Part of a kernel's output is
# still dirty in L2 when it ends, so written bytes come out below the algorithmic figure.  operand_cast = mean of
# its two launches (x: 254.6 MB, dy: 559.1 MB).
DRAM_TRAFFIC_S256 = {"igemm_fwd": 102976000 + 353129216, "igemm_dx": 205717760 + 154724608, "dw": 308411136 + 3284224,
                     "operand_cast": (205528320 + 49115136 + 411053824 + 147998976) // 2}
# algorithmic bytes per launch (each operand read once, each result written once)
def algorithmic_bytes(S, H, W, Cin, Cout):
    px = S * H * W
    return {"igemm_fwd": px * Cin * 2 + px * Cout * 4, "igemm_dx": px * Cout * 2 + px * Cin * 4,
            "dw": px * (Cin + Cout) * 2, "operand_cast": (px * Cin * 6 + px * Cout * 6) // 2}


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
CPU_IMAGES_PER_THREAD = 4    # both CPU legs (cpu_baseline and --impl reference) use this split, so they agree


def cpu_threads():
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    return max(1, min(n, 64))


def reference_checkout():
    """Path of an Aether-ML checkout to time verbatim ($AETHER_REFERENCE_ROOT, else the build container's mount), or
    None.  The reference is pure Python; it is never copied into this repository, so on a box without a checkout
    only the NumPy restatement (oracle/) can be timed."""
    for cand in (os.environ.get("AETHER_REFERENCE_ROOT"), "/root/reference"):
        if cand and os.path.exists(os.path.join(cand, "CNN", "models", "CNN_classes.py")):
            return cand
    return None


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


def cpu_reference_sample(root, images, min_seconds=0.0, max_passes=1):
    """Times the reference's own NumPy ``Conv_Layer`` (CNN/models/CNN_classes.py:5-125, imported from the checkout
    at `root`, unmodified): forward + backward on `images` images of the benchmark shape, float64 and one thread,
    which is how the reference runs.  Returns (TFLOP/s, seconds, passes)."""
    if root not in sys.path:
        sys.path.insert(0, root)
    from CNN.models.CNN_classes import Conv_Layer as RefConv
    rng = np.random.default_rng(4)
    s = SHAPE
    np.random.seed(4)
    layer = RefConv((s["H"], s["W"], s["Cin"]), num_filters=s["Cout"], filter_size=(s["f"], s["f"]), strides=(1, 1),
                    padding="same")
    x = rng.standard_normal((images, s["H"], s["W"], s["Cin"]))
    dy = rng.standard_normal((images, s["H"], s["W"], s["Cout"]))
    t0 = time.perf_counter()
    passes = 0
    while True:
        layer.forward(x, True)
        layer.backward(dy)
        passes += 1
        dt = time.perf_counter() - t0
        if dt >= min_seconds or passes >= max_passes:
            break
    fl = passes * conv_flops(images, s["H"], s["W"], s["Cin"], s["Cout"], s["f"])
    return fl / dt / 1e12, dt, passes


def cpu_baseline_block(min_seconds):
    """The CPU baseline of the benchmark line: the verbatim reference when a checkout is present (kind "reference",
    one thread, float64), else the NumPy restatement (kind "port") with the batch split over every host core in
    float32 -- the generous figure, also reported beside the verbatim one."""
    thr = cpu_threads()
    imgs = CPU_IMAGES_PER_THREAD * thr
    val, secs, passes = cpu_conv_sample(imgs, thr, min_seconds, 64)
    port = {"value": val, "unit": "TFLOP/s", "cores": thr, "kind": "port",
            "sample": "%d images of the workload shape (%d per worker thread), fwd+bwd %d times (%.1f s), NumPy einsum over "
                      "strided windows in float32 as in the reference, batch split over %d worker threads" % (imgs, CPU_IMAGES_PER_THREAD, passes, secs, thr)}
    root = reference_checkout()
    if root is None:
        return port
    rval, rsecs, rpasses = cpu_reference_sample(root, CPU_IMAGES_PER_THREAD, min_seconds, 64)
    return {"value": rval, "unit": "TFLOP/s", "cores": 1, "kind": "reference",
            "sample": "%d images of the workload shape, fwd+bwd %d times (%.1f s) through the reference's own NumPy "
                      "Conv_Layer (float64, one thread: np.einsum runs single-threaded)" % (CPU_IMAGES_PER_THREAD, rpasses, rsecs),
            "threaded_float32_port": port}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    s = SHAPE
    threads = cpu_threads()
    images = CPU_IMAGES_PER_THREAD * threads
    if args.warmup:
        cpu_conv_sample(images, threads, 1e9, args.warmup)
    # exactly `steps` passes over one sample; only the passes are timed (not the generation of the sample), as in
    # the cpu_baseline leg of the GPU arm
    val, dt, _ = cpu_conv_sample(images, threads, 1e9, args.steps)
    sample = ("%d images of the workload shape per step (%d per worker thread), NumPy einsum over strided windows in float32 "
              "(the reference's algorithm) on %d worker threads" % (images, CPU_IMAGES_PER_THREAD, threads))
    line = {
        "impl": "reference", "metric": "conv_fwd_bwd_tflops", "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    root = reference_checkout()
    if root is not None:       # the reference's own classes, as they run: one thread, float64 (reported beside the port)
        rval, rsecs, rpasses = cpu_reference_sample(root, CPU_IMAGES_PER_THREAD, 5.0, 8)
        line["verbatim_reference"] = {"value": rval, "unit": "TFLOP/s", "cores": 1, "kind": "reference",
                                      "sample": "%d images, fwd+bwd %d times (%.1f s), CNN/models/CNN_classes.py Conv_Layer, float64" % (CPU_IMAGES_PER_THREAD, rpasses, rsecs)}
    print(json.dumps(line))


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

    from aether_ml_b200 import dp
    world, rank, local = dp.init_from_env()
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
    h2d_bytes = (x_host.numel() + dy_host.numel()) * 4
    d2h_bytes = (y_out.numel() + dx_out.numel() + g_out.numel()) * 4

    # free the conv workload before the other blocks allocate theirs
    del xd, dyd, x, dy, y_out, dx_out, layer
    torch.cuda.empty_cache()
    sweep = run_sweep(args) if (world == 1 and not args.skip_sweep) else None
    train = None
    if not args.skip_train:
        torch.cuda.empty_cache()
        train = train_block(args, world, rank, local)

    if rank == 0:
        pk = peaks()
        fl_step = conv_flops(S, H, W, Cin, Cout, f)
        ms_step = ms_total / args.steps
        value = fl_step * world / (ms_step * 1e-3) / 1e12
        per_gemm = fl_step / 3.0
        tensor_peak = pk["sustained"] if ms_total > 1500 else pk["burst"]
        alg = algorithmic_bytes(S, H, W, Cin, Cout)
        per_kind = {}
        for k, (tot, n) in kinds.items():
            avg = tot / max(n, 1)
            per_step = avg * (2 if k == "operand_cast" else 1)          # two cast launches per step (x, dy)
            if k == "operand_cast":
                ach = alg[k] / (avg * 1e-3) / 1e9 if avg > 0 else None
                per_kind[k] = {"bound": "hbm", "achieved": ach, "peak": pk["hbm"], "unit": "GB/s",
                               "frac": ach / pk["hbm"] if ach else None, "bytes_per_launch": alg[k]}
            else:
                ach = per_gemm / (avg * 1e-3) / 1e12 if avg > 0 else None
                per_kind[k] = {"bound": "tensor", "achieved": ach, "peak": tensor_peak, "unit": "TFLOP/s",
                               "frac": ach / tensor_peak if ach else None, "flops_per_launch": per_gemm,
                               "hbm_gbs": alg[k] / (avg * 1e-3) / 1e9 if avg > 0 else None}
            per_kind[k].update({"launch_ms": avg, "ms_per_step": per_step, "timed_launches": n,
                                "traffic": DRAM_TRAFFIC_S256.get(k) if (S == 256 and args.mode == "bf16") else None})
        # dominant = the kernel kind with the largest share of the step (the two cast launches count together)
        dom = max(per_kind, key=lambda k: per_kind[k]["ms_per_step"])
        roof = dict(per_kind[dom])
        roof.update({"kernel": dom, "share_of_step": roof["ms_per_step"] / ms_step,
                     "traffic_unit": "bytes per launch (dram read + write, one-pass ncu capture of this workload)",
                     "peak_source": "%s (MEASURED_PEAKS.json: %s)" % (pk["source"], "hbm_gbs" if roof["bound"] == "hbm" else
                                                                      ("bf16_tflops_sustained" if ms_total > 1500 else "bf16_tflops")),
                     "timed_every": prof_stride})
        step_bytes = sum(alg[k] * (2 if k == "operand_cast" else 1) for k in alg)
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
                    "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes},
            "gpu_launches": int(launches),
            "roofline": roof,
            "roofline_kernels": per_kind,
            # what the whole step moves against what the memory system gives: the step is HBM-shaped at fp32 I/O
            "step_hbm": {"algorithmic_bytes_per_step": step_bytes, "achieved_gbs": step_bytes / (ms_step * 1e-3) / 1e9,
                         "frac_of_hbm_peak": step_bytes / (ms_step * 1e-3) / 1e9 / pk["hbm"],
                         "tensor_frac_at_hbm_peak": fl_step / (step_bytes / (pk["hbm"] * 1e9)) / 1e12 / pk["burst"]},
            "kernels": {k: {"total_ms": v[0], "launches": v[1], "avg_ms": v[0] / max(v[1], 1),
                            "tflops": (per_gemm / (v[0] / max(v[1], 1) * 1e-3) / 1e12) if (v[1] and k != "operand_cast" and v[0] > 0) else None}
                        for k, v in kinds.items()},
            "cpu_baseline": None if args.skip_cpu_baseline else cpu_baseline_block(10.0),
            "clocks": clocks,
        }
        if train is not None:
            out["train"] = train.pop("train")
            if "dp_check" in train:
                out["dp_check"] = train["dp_check"]
        if sweep is not None:
            out["sweep"] = sweep
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


# ----------------------------------------------------------------------------------- isolated conv sweep
SWEEP_SHAPES = [(256, 32, 32, 64, 64), (256, 16, 16, 128, 128), (256, 8, 8, 256, 256), (256, 56, 56, 64, 128)]


def hbm_ceiling_tflops(S, H, W, Cin, Cout, pk, tensor_peak):
    """min(tensor, HBM) roofline of one conv layer's fwd+bwd at fp32 I/O with each operand streamed once per GEMM:
    forward reads x writes y, dX reads dy writes dx, dW reads x and dy; filters are negligible."""
    px = S * H * W
    bytes_min = 4.0 * px * (Cin + Cout) * 3
    t = max(conv_flops(S, H, W, Cin, Cout, 3) / (tensor_peak * 1e12), bytes_min / (pk["hbm"] * 1e9))
    return conv_flops(S, H, W, Cin, Cout, 3) / t / 1e12


def run_sweep(args):
    """The isolated conv-layer sweep: batch 256, 3x3 stride 1 'same', four (H, W, Cin, Cout) shapes in bf16 and
    TF32, plus the first config (128, 32x32, 3 -> 32).  Each cell: 3 warm-up and 20 timed fwd+bwd steps queued back
    to back, CUDA events on the launching stream.  TF32 is judged against half the bf16 peak."""
    import torch
    from aether_ml_b200 import _lib
    from aether_ml_b200.layers import Conv_Layer
    pk = peaks()
    dev = torch.device("cuda", torch.cuda.current_device())
    cells = []
    todo = [(shape, mode) for mode in ("bf16", "tf32") for shape in SWEEP_SHAPES] + [((128, 32, 32, 3, 32), "bf16")]
    for (S, H, W, Cin, Cout), mode in todo:
        np.random.seed(99)
        layer = Conv_Layer((H, W, Cin), Cout, (3, 3), (1, 1), "same", math_mode=mode)
        g = torch.Generator(device="cuda").manual_seed(S + H + Cin)
        x = torch.randn((S, H, W, Cin), generator=g, device=dev) if Cin > 4 else torch.rand((S, H, W, Cin), generator=g, device=dev)
        dy = torch.randn((S, H, W, Cout), generator=g, device=dev)
        first = Cin <= 4
        l0 = _lib.launch_count()
        for _ in range(3):
            layer.forward(x, True)
            layer.backward(dy)
        launches = (_lib.launch_count() - l0) // 3
        torch.cuda.synchronize()
        iters = 20
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            layer.forward(x, True)
            layer.backward(dy)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
        fl = conv_flops(S, H, W, Cin, Cout, 3)
        tf = fl / (ms * 1e-3) / 1e12
        tensor_peak = pk["burst"] * (0.5 if mode == "tf32" else 1.0)
        ceil = hbm_ceiling_tflops(S, H, W, Cin, Cout, pk, tensor_peak)
        cells.append({"shape": [S, H, W, Cin, Cout], "mode": mode, "ms": ms, "tflops": tf, "launches_per_step": int(launches),
                      "pct_of_tensor_peak": 100.0 * tf / tensor_peak, "ceiling_tflops": ceil, "pct_of_ceiling": 100.0 * tf / ceil,
                      "note": "first config (a first layer: 12-byte pixels, HBM-bound)" if first else None})
        del layer, x, dy
        torch.cuda.empty_cache()
    if _lib.device_status() != 0:
        raise RuntimeError("a kernel abandoned a bounded wait: status %d" % _lib.device_status())
    return {"timing": "per cell 3 warm-up + 20 timed fwd+bwd steps back to back, CUDA events; TF32 against half the bf16 burst peak; "
                      "ceiling = min(tensor, HBM) roofline at fp32 I/O with each operand streamed once per GEMM", "cells": cells}


# ----------------------------------------------------------------------------------- training workload
def build_cnn(widen, math_mode, fuse=False, lean=False):
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
    m.finalize(flat=True, fuse=fuse, lean=lean and fuse)
    return m


def train_block(args, world, rank, local, widen=4, global_batch=4096, fuse=True, graph=True, steps=None, lean=True):
    """Training images/s of the 3-block CNN (widened 4x by default: channels 128/256/512, Dense 8192->1024->10) at a
    FIXED global batch sharded over the ranks (strong scaling).  One step = forward + loss gradient + backward +
    bucketed all-reduce of the flat gradient buffer (started during backward) + Adam; inputs resident on the device.
    Returns {"train": {...}, "dp_check": {...} (world > 1)} on every rank."""
    import torch
    import torch.distributed as dist
    from aether_ml_b200 import _lib, dp
    dev = torch.device("cuda", local)
    lo, hi = dp.shard_bounds(global_batch, rank, world)
    np.random.seed(7)                                   # same initial parameters on every rank
    model = build_cnn(widen, args.mode, fuse, lean)
    dp.attach(model, buckets=args.buckets)
    g = torch.Generator(device="cpu").manual_seed(3)
    X_host = torch.rand((global_batch, 32, 32, 3), generator=g)[lo:hi].contiguous().pin_memory()
    y_host = torch.randint(0, 10, (global_batch,), generator=g, dtype=torch.int32)[lo:hi].contiguous().pin_memory()
    X, y = X_host.to(dev), y_host.to(dev)

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    warm = max(args.warmup, 3)
    l0 = _lib.launch_count()
    for _ in range(warm):
        model.train_step(X, y)
    sync_all()
    launches_per_step = (_lib.launch_count() - l0) // warm
    if _lib.device_status() != 0:
        raise RuntimeError("a kernel abandoned a bounded wait: status %d" % _lib.device_status())

    # ---- data-parallel check (once): bucket-reduced buffer == sum of the ranks' own gradients
    dp_check = None
    if world > 1:
        held, model._bucket_of_layer = model._bucket_of_layer, {}      # a backward pass that starts no bucket
        out = model.forward(X, training=True)
        model.backward(out, y)
        model._bucket_of_layer = held
        own = model.flat_grads.clone()
        gathered = [torch.empty_like(own) for _ in range(world)]
        dist.all_gather(gathered, own)
        want = torch.stack(gathered).double().sum(dim=0)
        model.bucket_reducer.reduce_all()
        got = model.flat_grads.double()
        err = float((got - want).norm() / want.norm())
        differs = float((own.double() - want).norm() / want.norm())   # the check is not vacuous: one rank's gradient is not the sum
        dp_check = {"rel_l2_vs_allgather_sum": err, "own_gradient_vs_sum": differs, "elements": int(own.numel()),
                    "buckets": [[int(a), int(b)] for a, b, _ in model.bucket_reducer.buckets], "pass": bool(err <= 1e-6)}
        model.flat_grads.copy_(own)

    # ---- the all-reduce on its own (all buckets, nothing to overlap with)
    allreduce_ms = None
    if world > 1:
        sync_all()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        model.bucket_reducer.reduce_all()
        a0.record()
        for _ in range(5):
            model.bucket_reducer.reduce_all()
        a1.record()
        sync_all()
        t = torch.tensor([a0.elapsed_time(a1) / 5], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        allreduce_ms = float(t.item())
        model.flat_grads.zero_()

    step = model.train_step
    note = "eager"
    if graph:
        model.capture_train_step(X, y)
        note = model.capture_note
        step = model.train_step_graph
        for _ in range(3):
            step(X, y)
        sync_all()
    n_steps = steps or max(10, min(args.steps, 50))
    sampler = ClockSampler(local) if rank == 0 else None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    t_begin = time.perf_counter()
    e0.record()
    for _ in range(n_steps):
        step(X, y)
    e1.record()
    sync_all()
    t_end = time.perf_counter()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_step = float(ms.item()) / n_steps
    clocks = sampler.stop(t_begin, t_end) if sampler else None
    if _lib.device_status() != 0:
        raise RuntimeError("a kernel abandoned a bounded wait: status %d" % _lib.device_status())

    # ---- end to end: this step's shard uploaded from pinned memory, part of the result read back, every step
    def e2e_step():
        out = step(X_host.to(dev, non_blocking=True), y_host.to(dev, non_blocking=True))
        return out[:1].cpu()

    e2e_step()
    sync_all()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n_e2e = max(2, min(n_steps, 10))
    f0.record()
    for _ in range(n_e2e):
        e2e_step()
    f1.record()
    sync_all()
    ms2 = torch.tensor([f0.elapsed_time(f1)], device=dev)
    if world > 1:
        dist.all_reduce(ms2, op=dist.ReduceOp.MAX)
    e2e_ms = float(ms2.item()) / n_e2e
    train = {
        "metric": "train_images_per_s", "images_per_s": global_batch / (ms_step * 1e-3), "ms_per_step": ms_step,
        "steps": n_steps, "scaling": "strong", "global_batch": global_batch, "per_gpu_batch": hi - lo, "n_gpus": world,
        "workload": "train step of the CIFAR-shaped 3-block CNN%s, NHWC (32,32,3) ~ U[0,1), labels uniform in [0,10), Adam lr 1e-3 "
                    "decay 5e-5" % (" widened 4x (128/256/512, Dense 8192->1024->10)" if widen == 4 else ""),
        "params": int(model.flat_params.numel()), "fused_block_tails": bool(fuse), "cuda_graph": note,
        "lean": bool(lean and fuse),   # fp32 tensors read only as bf16 operand copies by our own next kernel are not written
        "allreduce_buckets": len(model.bucket_reducer.buckets) if world > 1 else 0,
        "allreduce_ms_alone": allreduce_ms, "launches_per_step": int(launches_per_step),
        "e2e_images_per_s": global_batch / (e2e_ms * 1e-3), "e2e_ms_per_step": e2e_ms,
        "h2d_bytes_per_step": (X_host.numel() * 4 + y_host.numel() * 4) * world, "d2h_bytes_per_step": 40 * world,
        "dtype": args.mode, "clocks": clocks,
    }
    res = {"train": train}
    if dp_check is not None:
        res["dp_check"] = dp_check
    model.release_graphs()      # before the process group goes: a graph with recorded collectives pins the communicator
    del model, X, y
    torch.cuda.empty_cache()
    return res


def run_train(args):
    """`--workload train|train_wide`: only the training block, as the line's headline metric."""
    import torch.distributed as dist
    from aether_ml_b200 import dp
    world, rank, local = dp.init_from_env()
    widen = 4 if args.workload == "train_wide" else 1
    global_batch = args.global_batch or (4096 if widen == 4 else 128)
    res = train_block(args, world, rank, local, widen=widen, global_batch=global_batch, fuse=args.fuse, graph=args.graph,
                      steps=args.steps, lean=args.lean)
    if rank == 0:
        t = res["train"]
        line = {"metric": "train_images_per_s", "value": t["images_per_s"], "unit": "images/s", "n_gpus": world,
                "steps": t["steps"], "warmup": max(args.warmup, 3), "ms_per_step": t["ms_per_step"], "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": args.mode, "data": "synthetic",
                "config": {"workload": t["workload"], "global_batch": global_batch, "per_gpu_batch": t["per_gpu_batch"],
                           "parallelism": "dp%d, %d all-reduce bucket(s) of the flat gradient buffer per step" % (world, t["allreduce_buckets"]),
                           "l2": "activations of a step (GBs) exceed the 126 MB L2", "params": t["params"],
                           "cuda_graph": t["cuda_graph"], "fused_block_tails": t["fused_block_tails"]},
                "e2e": {"value": t["e2e_images_per_s"], "unit": "images/s", "ms_per_step": t["e2e_ms_per_step"],
                        "h2d_bytes_per_step": t["h2d_bytes_per_step"], "d2h_bytes_per_step": t["d2h_bytes_per_step"]},
                "gpu_launches": t["launches_per_step"] * t["steps"], "train": t, "clocks": t["clocks"]}
        if "dp_check" in res:
            line["dp_check"] = res["dp_check"]
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_cell(args):
    """One cell of the sweep on its own: `--cell S,H,W,Cin,Cout` = fwd+bwd of one 3x3 stride-1 'same' Conv_Layer of that
    shape, `--warmup` + `--steps` passes, per-kernel-kind times from the library's event recorder.  The profiler
    captures of single kernels are taken on this command."""
    import ctypes as C
    import torch
    from aether_ml_b200 import _lib
    from aether_ml_b200.layers import Conv_Layer
    S, H, W, Cin, Cout = (int(v) for v in args.cell.split(","))
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    np.random.seed(99)
    layer = Conv_Layer((H, W, Cin), Cout, (3, 3), (1, 1), "same", math_mode=args.mode)
    g = torch.Generator(device="cuda").manual_seed(S + H + Cin)
    x = torch.randn((S, H, W, Cin), generator=g, device=dev)
    dy = torch.randn((S, H, W, Cout), generator=g, device=dev)
    for _ in range(args.warmup):
        layer.forward(x, True)
        layer.backward(dy)
    torch.cuda.synchronize()
    L = _lib.lib()
    L.aether_profile_reset()
    L.aether_profile_enable(1)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        layer.forward(x, True)
        layer.backward(dy)
    e1.record()
    torch.cuda.synchronize()
    kinds = {}
    for kind, name in enumerate(["igemm_fwd", "igemm_dx", "dw", "operand_cast"]):
        tot, n = C.c_double(0), C.c_int(0)
        L.aether_profile_read(kind, C.byref(tot), C.byref(n))
        kinds[name] = {"launches": n.value, "avg_ms": tot.value / max(n.value, 1)}
    L.aether_profile_enable(0)
    if _lib.device_status() != 0:
        raise RuntimeError("a kernel abandoned a bounded wait: status %d" % _lib.device_status())
    ms = e0.elapsed_time(e1) / max(args.steps, 1)
    print(json.dumps({"cell": [S, H, W, Cin, Cout], "mode": args.mode, "steps": args.steps, "ms_per_step": ms,
                      "tflops": conv_flops(S, H, W, Cin, Cout, 3) / (ms * 1e-3) / 1e12 if ms > 0 else None,
                      "note": "an event pair around every kernel: the step time is a few per cent above the sweep's", "kernels": kinds}))


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
    ap.add_argument("--graph", action="store_true", help="--workload train*: replay the step from a captured CUDA graph")
    ap.add_argument("--fuse", action="store_true",
                    help="--workload train*: fused block tails (finalize(fuse=True))")
    ap.add_argument("--lean", action="store_true",
                    help="--workload train*: with --fuse, do not write fp32 tensors that only our own next kernel reads (as bf16 copies)")
    ap.add_argument("--buckets", type=int, default=2, help="all-reduce buckets of the flat gradient buffer (1 = one all-reduce after backward)")
    ap.add_argument("--skip-train", action="store_true", help="default workload: omit the `train` block")
    ap.add_argument("--skip-sweep", action="store_true", help="default workload: omit the `sweep` block")
    ap.add_argument("--cell", default=None, metavar="S,H,W,Cin,Cout",
                    help="time fwd+bwd of one 3x3 'same' Conv_Layer of this shape (one GPU) and print its per-kernel times")
    args = ap.parse_args()
    # NCCL's in-switch reduction (NVLS) binds the ranks' buffers to an NVLink multicast object; a rank that dies while
    # bound can fault its peers' GPUs.  The collectives here (<= 40 MB) run without it unless the caller asks for it.
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    SHAPE["S"] = args.batch
    if args.impl == "reference":
        run_reference(args)
    elif args.cell:
        run_cell(args)
    elif args.workload == "conv":
        run_gpu(args)
    else:
        run_train(args)


if __name__ == "__main__":
    main()
