#!/usr/bin/env python
"""Benchmark: train images/s for one forward + backward + SGD step of ResNet-50 (batch 64 per GPU,
3x224x224 synthetic inputs, 1000 classes) through the mirrored executor and the C-ABI library.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload resnet50|vgg16|inceptionv3|densenet121|inceptionv4|lenet5|mlp]
    python bench.py --layer N,C,H,W,K,R,S,PADDING,STRIDE [--steps K]      one convolution layer on its own (profiling aid)

With N > 1 launch under torchrun (one rank per GPU); rank 0 prints one JSON line.
`--impl reference` times the CPU arm instead: the same graph evaluated by the numpy restatement of
the reference's operators (oracle/) on this box's host cores, on a bounded sample of the workload.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

# Algorithmic work per image of one training step (forward + backward-data + backward-filter of every
# convolution / matmul, 2 flops per multiply-add), computed from the graph by `step_flops` below.
WORKLOADS = {
    "resnet50": dict(batch=64, image=224, classes=1000, lr=0.01, dist="normal"),
    "vgg16": dict(batch=64, image=224, classes=1000, lr=0.01, dist="normal"),
    "inceptionv3": dict(batch=32, image=299, classes=1000, lr=0.01, dist="normal"),
    "densenet121": dict(batch=32, image=224, classes=1000, lr=0.01, dist="normal"),
    "inceptionv4": dict(batch=32, image=299, classes=1000, lr=0.01, dist="normal"),
    "lenet5": dict(batch=256, lr=0.05, dist="uniform"),
    "mlp": dict(batch=1000, lr=0.1, dist="uniform"),
}


# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) per launch of the contraction kernel, from one profiler
# capture: every distinct convolution layer of the workload at its benchmark batch launched on its own (`--layer WORKLOAD`,
# a few hundred MB on the device at a time), each layer's three launches weighted by how often the layer occurs in the graph.
# The full step holds tens of GB and its counters need several replay passes, so it is not captured whole; a layer's
# operands are the same size either way.  profiles/gemm3x_dram_traffic_resnet50_b64.md has the command and the table.
CONTRACTION_DRAM_BYTES_PER_LAUNCH = {("resnet50", "3xfp16"): 89.3e6}


def build_model(name, batch=None):
    from tinyflow_b200 import models
    cfg = dict(WORKLOADS[name])
    if batch is not None:
        cfg["batch"] = batch
    if name in ("resnet50", "vgg16", "inceptionv3", "densenet121", "inceptionv4"):
        return models.BUILDERS[name](batch=cfg["batch"], classes=cfg["classes"], image=cfg["image"]), cfg
    return models.BUILDERS[name](batch=cfg["batch"]), cfg


def step_flops(executor):
    """Algorithmic flops of one step: 2*M*N*K per matmul node, 2*N*K*P*Q*C*R*S per convolution node
    (forward, backward-data and backward-filter nodes each count once)."""
    total = 0
    shp = executor.node_to_shape_map
    for node in executor.topo_order:
        kind = type(node.op).__name__
        if kind == "MatMulOp":
            a, out = shp[node.inputs[0]], shp[node]
            k = a[0] if node.matmul_attr_trans_A else a[1]
            total += 2 * out[0] * out[1] * k
        elif kind in ("Convolution2DForwardOp", "Convolution2DBackwardOp"):
            x, w = shp[node.inputs[0]], shp[node.inputs[1]]
            y = shp[node] if kind == "Convolution2DForwardOp" else shp[node.inputs[2]]
            total += 2 * y[0] * y[1] * y[2] * y[3] * w[1] * w[2] * w[3]
    return total


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, gpu_index):
        super().__init__(daemon=True)
        self.gpu = gpu_index
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self.stop_flag = threading.Event()
        self.proc = None

    def run(self):
        q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
            "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + q, "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.proc.stdout:
            if self.stop_flag.is_set():
                break
            parts = [p.strip() for p in line.split(",")]
            try:
                self.samples.append(float(parts[0]))
                self.max_mhz = float(parts[1])
            except (ValueError, IndexError):
                continue
            for nm, val in zip(names, parts[2:]):
                if val.lower().startswith("active"):
                    self.reasons.add(nm)

    def finish(self):
        self.stop_flag.set()
        if self.proc is not None:
            self.proc.terminate()          # the exact process this sampler started
        s = sorted(self.samples)
        busy = [x for x in s if x > 0]
        med = busy[len(busy) // 2] if busy else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(s)}


def measured_peaks():
    path = os.path.join(REPO, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return d, "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


# ---------------------------------------------------------------------------------------------------
# CPU arm: the numpy restatement of the reference's operators on the same graph
# ---------------------------------------------------------------------------------------------------
def cpu_step_time(workload, sample_batch, repeats=1):
    """Seconds for one fp32 training step of `workload` at batch `sample_batch` on the host cores."""
    import numpy as np
    from oracle.graph_eval import OracleExecutor
    from tinyflow_b200 import autodiff as ad, models
    model, cfg = build_model(workload, batch=sample_batch)
    model.set_dropout(0.0)
    ex = ad.Executor(model.loss, model.y, cfg["lr"], None, None, None, optimizer="sgd")
    X, Y = models.synthetic_batch(model, seed=1234, input_dist=cfg["dist"])
    feed = {model.X: X, model.y_: Y}
    feed.update(model.init_params(seed=123))
    orc = OracleExecutor(ex.topo_order, np.float32)
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        orc.run(feed)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return best


def cpu_threads():
    try:
        from threadpoolctl import threadpool_info
        n = max([p.get("num_threads", 1) for p in threadpool_info()] + [1])
    except Exception:
        n = 1
    return n, len(os.sched_getaffinity(0))


def pin_blas_threads():
    """Gives the BLAS behind numpy every usable core (at most the 64 OpenBLAS is built for), whatever the launcher put
    into OMP_NUM_THREADS (torchrun sets it to 1).  Call before numpy is imported; repeated through threadpoolctl for
    a BLAS that is already loaded."""
    want = max(1, min(len(os.sched_getaffinity(0)), 64))
    for var in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        os.environ[var] = str(want)
    try:
        import numpy  # noqa: F401
        from threadpoolctl import threadpool_limits
        threadpool_limits(limits=want)
    except Exception:
        pass
    return want


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    pin_blas_threads()
    import numpy as np  # noqa: F401  (loads the BLAS whose thread count is reported)
    workload = args.workload
    cfg = WORKLOADS[workload]
    sample = {"resnet50": 4, "vgg16": 2, "inceptionv3": 2, "densenet121": 2, "inceptionv4": 2}.get(workload, cfg["batch"])
    blas_threads, cores = cpu_threads()
    for _ in range(args.warmup if workload in ("mlp", "lenet5") else min(args.warmup, 1)):
        cpu_step_time(workload, sample)
    t0 = time.perf_counter()
    per_step = [cpu_step_time(workload, sample) for _ in range(args.steps)]
    wall = time.perf_counter() - t0
    sec = sum(per_step) / len(per_step)
    value = sample / sec
    line = {
        "impl": "reference", "metric": "train images/sec (fwd+bwd+SGD) %s" % workload, "value": value, "unit": "images/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1000.0 * cfg["batch"] / sample,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "%s b%d fp32 fwd+bwd+SGD" % (workload, cfg["batch"]), "sample": "one step at batch %d (images/s does not depend on the batch for this arm)" % sample},
        "cpu_baseline": {"value": value, "unit": "images/s", "cores": blas_threads, "kind": "port",
                         "sample": "numpy fp32 restatement of the reference operators, batch %d, %d steps, %d BLAS threads on %d usable cores, %.1f s" % (sample, args.steps, blas_threads, cores, wall)},
        "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    from tinyflow_b200._base import _LIB
    assert not _LIB.loaded, "the CPU arm must not map the CUDA library"
    print(json.dumps(line))
    return 0


# ---------------------------------------------------------------------------------------------------
# one layer on its own (profiling aid)
# ---------------------------------------------------------------------------------------------------
def conv_layers_of(workload):
    """Distinct convolution layers of a workload's graph at its benchmark batch: [(N, C, H, W, K, R, S, padding, stride, count)]."""
    from tinyflow_b200 import autodiff as ad
    model, cfg = build_model(workload)
    ex = ad.Executor(model.loss, model.y, cfg["lr"], None, None, None, optimizer="sgd")
    shapes = {model.X: model.input_shape, model.y_: model.label_shape}
    shapes.update({var: tuple(shape) for var, shape in model.param_shapes.items()})
    ex.infer_shape(shapes)
    found = {}
    for node in ex.topo_order:
        if type(node.op).__name__ == "Convolution2DForwardOp":
            x, w = ex.node_to_shape_map[node.inputs[0]], ex.node_to_shape_map[node.inputs[1]]
            key = (*x, w[0], w[2], w[3], node.padding, node.u)
            found[key] = found.get(key, 0) + 1
    return [(*k, c) for k, c in found.items()]


def run_layer(args):
    """One convolution layer (or, given a workload name, each distinct layer of that workload in turn) on its own."""
    import ctypes
    import numpy as np
    from tinyflow_b200 import gpu_op, ndarray
    from tinyflow_b200._base import _LIB
    if args.layer in WORKLOADS:
        layers = conv_layers_of(args.layer)
    else:
        f = args.layer.split(",")
        layers = [(*(int(v) for v in f[:7]), f[7], int(f[8]), 1)]
    ctx = ndarray.gpu(0)
    stream = gpu_op.create_cudaStream()
    cudnn = gpu_op.create_cudnnHandle(stream)
    rng = np.random.RandomState(0)
    out = []
    for (N, C, H, W, K, R, S, padding, stride, count) in layers:
        x = ndarray.array(rng.randn(N, C, H, W).astype(np.float32), ctx)
        w = ndarray.array((rng.randn(K, C, R, S) * np.sqrt(2.0 / (C * R * S))).astype(np.float32), ctx)
        out_shape, cell = gpu_op.convolution_2d_forward_get_out_shape((N, C, H, W), (K, C, R, S), "NCHW", padding, stride, stride)
        y, dy = ndarray.empty(out_shape, ctx), ndarray.array(rng.randn(*out_shape).astype(np.float32), ctx)
        dx, dw = ndarray.empty((N, C, H, W), ctx), ndarray.empty((K, C, R, S), ctx)

        def passes():
            gpu_op.convolution_2d_forward(x, w, y, cell, cudnn, stream)
            if C >= 16:
                gpu_op.convolution_backward_data(x, dy, w, dx, cell, cudnn, stream)
            gpu_op.convolution_backward_filter(x, dy, w, dw, cell, cudnn, stream)

        for _ in range(max(args.warmup, 1)):
            passes()
        gpu_op.device_synchronize()
        _LIB.TfKernelTimingEnable(2)
        for _ in range(args.steps):
            passes()
        gpu_op.device_synchronize()
        report = ctypes.create_string_buffer(1 << 16)
        _LIB.TfKernelTimingReport(report, len(report))
        _LIB.TfKernelTimingEnable(0)
        rows = json.loads(report.value.decode() or "[]")
        for r in rows:
            t = r["ms"] / max(r["launches"], 1)
            r.update(us_per_launch=1000.0 * t, tflops=(r["flops"] / r["launches"] / t / 1e9 if t and r["flops"] else 0.0),
                     gbs=(r["bytes"] / r["launches"] / t / 1e6 if t and r["bytes"] else 0.0))
        out.append({"layer": "%d,%d,%d,%d,%d,%d,%d,%s,%d" % (N, C, H, W, K, R, S, padding, stride), "count_in_graph": count,
                    "passes": 3 if C >= 16 else 2, "kernels": rows})
        del x, w, y, dy, dx, dw
    print(json.dumps({"layers": out, "arithmetic": gpu_op.tensor_arithmetic(), "steps": args.steps, "warmup": max(args.warmup, 1)}))
    return 0


def run_matmul(args):
    import ctypes
    import numpy as np
    from tinyflow_b200 import gpu_op, ndarray
    from tinyflow_b200._base import _LIB
    M, K, N = (int(v) for v in args.matmul.split(","))
    ctx = ndarray.gpu(0)
    stream = gpu_op.create_cudaStream()
    cublas = gpu_op.create_cublasHandle(stream)
    rng = np.random.RandomState(0)
    A, B, C = ndarray.array(rng.randn(M, K).astype(np.float32), ctx), ndarray.array(rng.randn(K, N).astype(np.float32), ctx), ndarray.empty((M, N), ctx)
    out = {"matmul": [M, K, N], "steps": args.steps, "modes": {}}
    for name, path, arith in (("3xfp16", 2, "3xfp16"), ("3xtf32", 2, "3xtf32"), ("fp32 CUDA cores", 1, "3xfp16")):
        gpu_op.set_contraction_path(path)
        gpu_op.set_tensor_arithmetic(arith)
        reps = args.steps if path == 2 else max(1, args.steps // 4)
        try:
            for _ in range(3):
                gpu_op.matrix_multiply(A, False, B, False, C, cublas, stream)
            gpu_op.device_synchronize()
            _LIB.TfKernelTimingEnable(1)
            for _ in range(reps):
                gpu_op.matrix_multiply(A, False, B, False, C, cublas, stream)
            gpu_op.device_synchronize()
            report = ctypes.create_string_buffer(1 << 14)
            _LIB.TfKernelTimingReport(report, len(report))
            _LIB.TfKernelTimingEnable(0)
        finally:
            gpu_op.set_contraction_path(0)
            gpu_op.set_tensor_arithmetic("3xfp16")
        rows = [r for r in json.loads(report.value.decode() or "[]") if r["flops"] > 0]
        ms = sum(r["ms"] for r in rows) / max(reps, 1)
        alg = 2.0 * M * N * K / (ms / 1000.0) / 1e12 if ms else 0.0
        out["modes"][name] = {"ms": ms, "algorithmic_tflops": alg, "issued_tflops": 3 * alg if path == 2 else alg}
    print(json.dumps(out))
    return 0


# ---------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--workload", default="resnet50", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--memory-plan", default="none", choices=["none", "vdnn-conv", "vdnn-all"],
                    help="replay a swap/release plan (reference message format) during every step; not the headline configuration")
    ap.add_argument("--batch", type=int, default=None, help="per-GPU batch override (profiling on a small case; not the headline configuration)")
    ap.add_argument("--layer", default=None, metavar="N,C,H,W,K,R,S,PADDING,STRIDE | WORKLOAD",
                    help="time the three passes of ONE convolution layer on its own (e.g. 64,256,14,14,256,3,3,SAME,1), or of every "
                         "distinct layer of a workload one after the other (e.g. resnet50), and print a per-kernel JSON table: the "
                         "small cases profiler captures run on; not the headline configuration")
    ap.add_argument("--matmul", default=None, metavar="M,K,N",
                    help="time one M x K by K x N product in both arithmetic modes of the tensor path (3xFP16, 3xTF32) and on the "
                         "exact-fp32 CUDA-core kernel; prints a JSON line (measures the issued tensor rate each mode reaches)")
    args = ap.parse_args()
    if args.layer:
        return run_layer(args)
    if args.matmul:
        return run_matmul(args)
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        return run_reference_arm(args)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus %d needs a torchrun launch with %d ranks" % (args.gpus, args.gpus))
    physical_gpu = local_rank
    if world > 1:
        # one process per GPU; the executor addresses its GPU as gpu(0), as the reference hard-codes
        os.environ["CUDA_VISIBLE_DEVICES"] = str(local_rank)

    import ctypes
    import numpy as np
    import torch
    from tinyflow_b200 import autodiff as ad, gpu_op, models, ndarray
    from tinyflow_b200._base import _LIB, check_call

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); use --impl reference for the CPU arm")
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda:0"))
        id_path = "/tmp/tinyflow_b200_nccl_id_%s" % os.environ.get("MASTER_PORT", "0")
        check_call(_LIB.TfDpInit(rank, world, id_path.encode()))

    model, cfg = build_model(args.workload, batch=args.batch)
    model.set_dropout({"resnet50": 0.5, "vgg16": 0.5, "inceptionv3": 0.8, "densenet121": 0.2, "inceptionv4": 0.8}.get(args.workload, 0.0))
    import queue
    control = queue.Queue()
    ex = ad.Executor(model.loss, model.y, cfg["lr"], control, None, None, optimizer="sgd")
    ctx = ndarray.gpu(0)
    Xn, Yn = models.synthetic_batch(model, seed=1234, rank=rank, input_dist=cfg["dist"])
    params = model.init_params(seed=123)          # identical on every rank
    feed = {n: ndarray.array(v, ctx) for n, v in params.items()}
    Xd, Yd = ndarray.array(Xn, ctx), ndarray.array(Yn, ctx)
    # pinned host staging for the end-to-end arm
    Xh, Yh = ndarray.array(Xn, ndarray.cpu(0)), ndarray.array(Yn, ndarray.cpu(0))
    batch = cfg["batch"]

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def flush_dp():
        # end of a data-parallel step: sends the last, partly filled gradient bucket and makes the compute stream
        # wait for every applied update, so the next forward pass reads the new weights
        if world > 1:
            check_call(_LIB.TfDpFlush(ex.cudaStream))

    def step_resident(fd):
        fd[model.X], fd[model.y_] = Xd, Yd
        loss, nxt = ex.run(fd)
        flush_dp()
        return loss, nxt

    # End-to-end arm: every step uploads its inputs from pinned host memory and reads its loss back.  The upload of
    # step k+1 runs on a side stream from a helper thread while step k computes (the swap threads of the reference's
    # executor use DLArrayCopyFromTo the same way): two device buffers alternate, the helper's call returns when its
    # copy has completed, and the step that consumes a buffer joins the helper first.
    in_bufs = [(ndarray.empty(Xn.shape, ctx), ndarray.empty(Yn.shape, ctx)) for _ in range(2)]
    copy_stream = gpu_op.create_cudaStream()
    upload = {"thread": None, "k": 0}

    def start_upload(slot):
        def work():
            Xh.copyto(in_bufs[slot][0], copy_stream)
            Yh.copyto(in_bufs[slot][1], copy_stream)
        t = threading.Thread(target=work, daemon=True)
        t.start()
        upload["thread"] = t

    def step_e2e(fd):
        k = upload["k"]
        if upload["thread"] is None:
            start_upload(k & 1)
        upload["thread"].join()                       # this step's inputs are on the device
        fd[model.X], fd[model.y_] = in_bufs[k & 1]
        start_upload((k + 1) & 1)                     # next step's inputs travel while this step computes
        upload["k"] = k + 1
        loss, nxt = ex.run(fd)
        flush_dp()
        return loss.asnumpy(), nxt                    # device -> host read of the loss: the step has finished

    plan_info = None
    for w in range(args.warmup):
        if w == 1 and args.memory_plan != "none":          # shapes are known after the first step
            from tinyflow_b200 import memory_plan
            plan = memory_plan.vdnn_plan(ex, policy=args.memory_plan.split("-")[1])
            out_bytes = sum(4 * int(np.prod(ex.node_to_shape_map[ex.topo_order[t]])) for t, _w, _s, to_gpu in plan[0] if not to_gpu)
            # the swap traffic's own roofline: bytes each way over the measured pinned-memory link rate (the two directions
            # run on separate copy engines, so the bound is one direction's bytes)
            probe_h, probe_d = ndarray.empty((64 * 1024 * 1024,), ndarray.cpu(0)), ndarray.empty((64 * 1024 * 1024,), ctx)
            probe_h.copyto(probe_d, copy_stream)
            t0 = time.perf_counter()
            for _ in range(4):
                probe_h.copyto(probe_d, copy_stream)
            h2d = 4 * 256 * 1024 * 1024 / (time.perf_counter() - t0) / 1e9
            t0 = time.perf_counter()
            for _ in range(4):
                probe_d.copyto(probe_h, copy_stream)
            d2h = 4 * 256 * 1024 * 1024 / (time.perf_counter() - t0) / 1e9
            del probe_h, probe_d
            plan_info = {"policy": args.memory_plan, "swapped_tensors": len(plan[0]) // 2, "released_tensors": len(plan[1]),
                         "bytes_away_at_peak": int(memory_plan.check_plan(ex, plan)), "bytes_each_way_per_step": int(out_bytes),
                         "host_link_gbs": {"h2d": h2d, "d2h": d2h}, "host_link_bound_ms": out_bytes / 1e6 / min(h2d, d2h)}
            control.put(plan)
        loss, feed = step_resident(feed)
    if args.memory_plan != "none" and plan_info is None:
        raise SystemExit("--memory-plan needs --warmup >= 2")
    barrier()
    flops = step_flops(ex)

    # ---- timed region 1: inputs resident in HBM, device-timed with CUDA events on the executor's stream
    stream_ptr = ctypes.cast(ex.cudaStream, ctypes.POINTER(ctypes.c_void_p)).contents.value
    ext = torch.cuda.ExternalStream(stream_ptr)
    sampler = ClockSampler(physical_gpu)
    sampler.start()
    time.sleep(0.3)
    n0 = gpu_op.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_wall0 = time.perf_counter()
    e0.record(ext)
    for _ in range(args.steps):
        loss, feed = step_resident(feed)
    e1.record(ext)
    barrier()
    wall = time.perf_counter() - t_wall0
    dev_ms = e0.elapsed_time(e1)
    launches = gpu_op.launch_count() - n0

    # ---- the same K steps again with a CUDA-event pair around every launch of the contraction kernels (the roofline
    # figure).  Kept out of the region above because an event record between two kernels serialises them the ordinary
    # way and so takes the dependent-launch overlap away from every instrumented launch (about 2 % of the step).
    _LIB.TfKernelTimingEnable(1)
    barrier()
    t_i0 = time.perf_counter()
    for _ in range(args.steps):
        loss, feed = step_resident(feed)
    barrier()
    instrumented_ms = (time.perf_counter() - t_i0) * 1000.0 / args.steps
    report = ctypes.create_string_buffer(1 << 16)
    _LIB.TfKernelTimingReport(report, len(report))
    _LIB.TfKernelTimingEnable(0)
    clocks = sampler.finish()
    kernel_rows = json.loads(report.value.decode() or "[]")
    final_loss = float(loss.asnumpy()[0])

    # ---- timed region 2: end to end through the public API with host buffers
    for _ in range(2):
        _, feed = step_e2e(feed)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        lv, feed = step_e2e(feed)
    barrier()
    e2e_s = time.perf_counter() - t0
    upload["thread"].join()                           # the look-ahead upload of a step that is never run

    # ---- untimed extra steps with every instrumented kernel timed: the per-kernel table
    _LIB.TfKernelTimingEnable(2)
    prof_steps = 2
    for _ in range(prof_steps):
        loss, feed = step_resident(feed)
    barrier()
    _LIB.TfKernelTimingReport(report, len(report))
    _LIB.TfKernelTimingEnable(0)
    all_rows = json.loads(report.value.decode() or "[]")
    for r in all_rows:
        r["ms_per_step"] = r.pop("ms") / prof_steps
        r["launches_per_step"] = r.pop("launches") / prof_steps
        r["gflop_per_step"] = r.pop("flops") / prof_steps / 1e9
        r["gb_per_step"] = r.pop("bytes") / prof_steps / 1e9
        t = r["ms_per_step"] / 1000.0
        r["tflops"] = r["gflop_per_step"] / 1e3 / t if t > 0 else 0.0
        r["gbs"] = r["gb_per_step"] / t if t > 0 else 0.0

    if os.environ.get("TINYFLOW_KERNEL_TABLE") and rank == 0:
        json.dump(all_rows, open(os.environ["TINYFLOW_KERNEL_TABLE"], "w"), indent=0)

    # Data-parallel correctness bit: every rank must hold bit-identical weights after the timed steps.  Each weight
    # tensor is digested (sum of its 32-bit patterns, and its float64 sum) and the digests' minimum and maximum over
    # the ranks are compared.
    dp_identical = None
    if dist is not None:
        digest = []
        for var in model.param_shapes:
            w = feed[var].asnumpy()
            digest += [float(w.view(np.uint32).astype(np.uint64).sum() % (1 << 52)), float(w.astype(np.float64).sum())]
        lo = torch.tensor(digest, dtype=torch.float64, device="cuda:0")
        hi = lo.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        dp_identical = bool(torch.equal(lo, hi))
    dp_stats = None
    if world > 1:
        c = [ctypes.c_longlong(0) for _ in range(4)]
        check_call(_LIB.TfDpStats2(*[ctypes.byref(v) for v in c]))
        dp_stats = {"bytes_reduced": c[0].value, "allreduces": c[1].value, "update_launches": c[2].value, "early_bucket_closes": c[3].value,
                    "note": "totals of this rank since TfDpInit (warm-up, timed and instrumented steps)"}

    ms = torch.tensor([max(dev_ms, 0.0), wall * 1000.0, e2e_s * 1000.0], dtype=torch.float64, device="cuda:0")
    if dist is not None:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    dev_ms, wall_ms, e2e_ms = [float(x) for x in ms.tolist()]
    # the CPU can run ahead of the GPU, never behind the device-side events by more than the queue depth:
    # the slower of the two clocks is the honest step time
    step_ms = max(dev_ms, wall_ms) / args.steps
    value = world * batch / (step_ms / 1000.0)
    e2e_value = world * batch / (e2e_ms / 1000.0 / args.steps)

    peaks, peak_kind = measured_peaks()
    roofline = None
    if kernel_rows:
        top = max(kernel_rows, key=lambda r: r["ms"])
        total_ms = sum(r["ms"] for r in kernel_rows)
        if top["flops"] > 0:
            # 3xFP16 issues three tensor-core MMAs per algorithmic multiply-add; the denominator is the measured 16-bit
            # tensor rate (fp16 runs at the bf16 rate), sustained figure because the kernel runs inside a long step
            peak = peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])
            ach = top["flops"] / (top["ms"] / 1000.0) / 1e12
            roofline = {"bound": "tensor", "kernel": top["name"], "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak,
                        "traffic": CONTRACTION_DRAM_BYTES_PER_LAUNCH.get((args.workload, gpu_op.tensor_arithmetic())) if args.batch is None else None,
                        "traffic_source": "DRAM read+write bytes per launch: profiler capture of each distinct convolution layer of this workload at this batch, launched on its own, weighted by its count in the graph (not captured in this run)",
                        "launches": top["launches"], "avg_us": 1000.0 * top["ms"] / max(top["launches"], 1),
                        "issued": 3.0 * ach, "issued_frac": 3.0 * ach / peak,
                        "timed_over": "%d steps repeated right after the timed region with an event pair around each launch (%.3f ms per step there)" % (args.steps, instrumented_ms),
                        "peak_source": "%s bf16 sustained (fp16 inputs run at the same rate); achieved/frac count algorithmic flops, issued/issued_frac the three fp16 products 3xFP16 spends per multiply-add (what the tensor-pipe counter sees)" % peak_kind,
                        "share_of_timed_kernels": top["ms"] / total_ms if total_ms else None}
        else:
            peak = peaks["hbm_gbs"]
            ach = top["bytes"] / (top["ms"] / 1000.0) / 1e9
            roofline = {"bound": "hbm", "kernel": top["name"], "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                        "traffic": None, "launches": top["launches"], "avg_us": 1000.0 * top["ms"] / max(top["launches"], 1),
                        "peak_source": peak_kind + " copy bandwidth"}

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        sample = {"resnet50": 4, "vgg16": 2, "inceptionv3": 2, "densenet121": 2, "inceptionv4": 2}.get(args.workload, batch)
        t = cpu_step_time(args.workload, sample)
        threads, cores = cpu_threads()
        cpu_baseline = {"value": sample / t, "unit": "images/s", "cores": threads, "kind": "port",
                        "sample": "numpy fp32 restatement of the reference operators, one step at batch %d (%.1f s), %d BLAS threads on %d usable cores" % (sample, t, threads, cores)}

    if rank == 0:
        line = {
            "metric": "train images/sec (fwd+bwd+SGD) %s" % args.workload, "value": value, "unit": "images/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "%s b%d/GPU %s fp32 fwd+bwd+SGD" % (args.workload, batch, "x".join(str(d) for d in model.input_shape[1:])),
                       "global_batch": world * batch, "parallelism": "dp%d" % world, "l2": "per-step working set (GBs of activations) exceeds the 126 MB L2",
                       "dropout": (model.dropout_nodes[0].dropout if model.dropout_nodes else 0.0), "device_ms_per_step": dev_ms / args.steps, "host_ms_per_step": wall_ms / args.steps,
                       "algorithmic_tflop_per_step": flops / 1e12, "final_loss": final_loss, "memory_plan": plan_info,
                       "passive_swap_ins": ex.passive_swap_in, "arithmetic": gpu_op.tensor_arithmetic(),
                       "dp_weights_identical": dp_identical, "dp_stats": dp_stats},
            "e2e": {"value": e2e_value, "unit": "images/s", "h2d_bytes_per_step": int(Xn.nbytes + Yn.nbytes), "d2h_bytes_per_step": 4},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "roofline": roofline,
            "cpu_baseline": cpu_baseline,
            "kernels": sorted(all_rows, key=lambda r: -r["ms_per_step"])[:16],
        }
        print(json.dumps(line))
    if dist is not None:
        _LIB.TfDpShutdown()
        dist.destroy_process_group()
    sys.stdout.flush()
    return 0


if __name__ == "__main__":
    sys.exit(main())
