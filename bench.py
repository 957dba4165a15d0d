#!/usr/bin/env python
"""Benchmark of the quantized operator hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME] [--lanes S] [--grid-cap G]

One JSON line on stdout (rank 0).  A "step" is one pass of the hot path over one batch of seeded synthetic input.
The default workload is the whole MobileNetV2-1.0 224x224 uint8 graph on ONE batch of 256 images: at N GPUs
(torchrun, one process per GPU) the batch is partitioned into contiguous slices of 256 / N images, every rank runs
its slice, there is no collective on the data path, and only the 256 x 1000 logits are gathered on rank 0
(metric: images/s of the whole job; "scaling": "strong").  Single-operator workloads (--workload depthwise3x3_s1 ...)
report HBM GB/s or int8 TOPS of that operator.

`value` is measured with inputs resident in HBM (CUDA events on the library's streams); `e2e` is the same metric
through the operator-list C ABI with HOST buffers: host->device copy of every step's images, the graph, the
device->host copy of the logits and, at N > 1, the gather of all ranks' logits on rank 0 inside the timed region.
A rank runs several operator lists ("lanes", each with its own stream, buffers and CUDA graph) and hands
successive steps to them in turn; the persistent kernels of a lane launch on a share of the SMs (context option
grid_cap, a quarter of the GPU by default), so that kernels of four different steps run side by side and the latency
of the small layers is hidden (--lanes 3 --grid-cap 0 gives whole-GPU kernels that only overlap at their tails).
`--impl reference` times the CPU oracle (the reference has no CPU implementation of these operators and its OpenCL
path cannot run on this machine) on a bounded sample of the same workload, with all host threads.
"""
import argparse
import ctypes as C
import gc
import importlib
import importlib.util
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "cl-eden-kernel_b200")
sys.path.insert(0, ROOT)

DEFAULT_WORKLOAD = "mobilenetv2_u8_b256"
GLOBAL_BATCH = 256
WORKLOAD_TEXT = "MobileNetV2-1.0 224x224 uint8 graph (per-channel int8 weights), one batch of 256 images partitioned over the GPUs"

# DRAM traffic of the graph's kernels from one ncu pass (dram__bytes_read.sum + dram__bytes_write.sum per launch) over one
# step of the batch-256 graph (profiles/mobilenetv2_graph_launch_list.md), as measured bytes / algorithmic bytes per kernel
# family.  Below 1 because the 126 MB L2 still holds part of every layer's output when the next kernel reads it; the
# tensors are activations, so the traffic of a smaller per-rank batch is at most this share of its algorithmic bytes.
NCU_TRAFFIC_RATIO = {"tc_gemm_kernel": 0.653, "dw3x3_ring_kernel": 0.745, "conv3x3c3_kernel": 0.617, "add_kernel_lut2": 0.671,
                     "avgpool_vec4_kernel": 0.986}


def load_package():
    name = "cl_eden_kernel_b200"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, os.path.join(PKG, "__init__.py"), submodule_search_locations=[PKG])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def load_plain(modname):
    """A module of the package directory loaded on its own (descriptors, workloads, graph builder): the CPU arm uses
    these without importing the package, i.e. without loading the CUDA library."""
    if PKG not in sys.path:
        sys.path.insert(0, PKG)
    return importlib.import_module(modname)


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": d.get("hbm_gbs", 6650.0), "bf16_tflops": d.get("bf16_tflops", 1590.0), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []
        self.first = 0

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.gpu)], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def wait_first_sample(self, timeout=10.0):
        t0 = time.perf_counter()
        while self.proc and not self.lines and time.perf_counter() - t0 < timeout and self.proc.poll() is None:
            time.sleep(0.01)

    def mark(self):
        """Samples taken before this call are dropped from the summary (they precede the timed regions)."""
        self.first = len(self.lines)

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.1)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines[self.first:]:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


class Cuda:
    """The few runtime calls the benchmark needs on the library's own streams (events, graph capture)."""

    def __init__(self):
        rt = C.CDLL("libcudart.so")
        rt.cudaEventCreate.argtypes = [C.POINTER(C.c_void_p)]
        rt.cudaEventRecord.argtypes = [C.c_void_p, C.c_void_p]
        rt.cudaEventSynchronize.argtypes = [C.c_void_p]
        rt.cudaEventElapsedTime.argtypes = [C.POINTER(C.c_float), C.c_void_p, C.c_void_p]
        rt.cudaStreamWaitEvent.argtypes = [C.c_void_p, C.c_void_p, C.c_uint]
        self.rt = rt

    def event(self):
        e = C.c_void_p()
        assert self.rt.cudaEventCreate(C.byref(e)) == 0
        return e

    def record(self, e, stream):
        assert self.rt.cudaEventRecord(e, stream) == 0

    def stream_wait(self, stream, e):
        assert self.rt.cudaStreamWaitEvent(stream, e, 0) == 0

    def elapsed_ms(self, e0, e1):
        ms = C.c_float()
        assert self.rt.cudaEventSynchronize(e1) == 0
        assert self.rt.cudaEventElapsedTime(C.byref(ms), e0, e1) == 0
        return ms.value

    def capture(self, stream, fn):
        """Runs fn() with `stream` in capture mode and returns an executable graph of what it enqueued (or None)."""
        rt = self.rt
        rt.cudaStreamBeginCapture.argtypes = [C.c_void_p, C.c_int]
        rt.cudaStreamEndCapture.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
        rt.cudaGraphInstantiate.argtypes = [C.POINTER(C.c_void_p), C.c_void_p, C.c_ulonglong]
        rt.cudaGraphDestroy.argtypes = [C.c_void_p]
        if rt.cudaStreamBeginCapture(stream, 2) != 0:      # relaxed: the library's host-side calls stay legal
            return None
        try:
            fn()
        finally:
            graph = C.c_void_p()
            st = rt.cudaStreamEndCapture(stream, C.byref(graph))
        if st != 0 or not graph:
            return None
        exe = C.c_void_p()
        st = rt.cudaGraphInstantiate(C.byref(exe), graph, 0)
        rt.cudaGraphDestroy(graph)
        return exe if st == 0 and exe else None

    def launch_graph(self, exe, stream):
        self.rt.cudaGraphLaunch.argtypes = [C.c_void_p, C.c_void_p]
        assert self.rt.cudaGraphLaunch(exe, stream) == 0

    def destroy_graph(self, exe):
        self.rt.cudaGraphExecDestroy.argtypes = [C.c_void_p]
        self.rt.cudaGraphExecDestroy(exe)


def dist_env():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))


# ---------------------------------------------------------------------------------------------------
# Single-operator configurations (BASELINE configs 1-4), timed over rotating buffer sets larger than L2
# ---------------------------------------------------------------------------------------------------
def op_configs(cases):
    return {
        "conv3x3_1x56x56x64": ("conv2d", lambda: cases.conv_case(seed=0), "tensor"),
        "conv3x3_256x56x56x64": ("conv2d", lambda: cases.conv_case(seed=0, n=256), "tensor"),
        "depthwise3x3_s1_64x112x112x32": ("depthwise", lambda: cases.depthwise_case(seed=0, n=64), "hbm"),
        "depthwise3x3_s2_64x112x112x32": ("depthwise", lambda: cases.depthwise_case(seed=0, n=64, stride=2), "hbm"),
        "fc_1x4096x4096": ("fully_connected", lambda: cases.fc_case(seed=0, m=1, k=4096, n=4096), "hbm"),
        "fc_256x1024x1024": ("fully_connected", lambda: cases.fc_case(seed=0, m=256, k=1024, n=1024), "tensor"),
        "fc_4096x4096x4096": ("fully_connected", lambda: cases.fc_case(seed=0, m=4096, k=4096, n=4096), "tensor"),
        "deconv4x4_s2_8x64x64x128": ("deconv", lambda: cases.deconv_case(seed=0, n=8, h=64, w=64), "tensor"),
        # the MobileNetV2 layers that dominate the graph step, as stand-alone workloads for profiling
        "mnv2_expand_256x112x112x16to96": ("conv2d", lambda: cases.conv_case(seed=0, n=256, h=112, w=112, cin=16, cout=96, k=1, per_channel=True, out_scale=0.0235, out_zp=0), "hbm"),
        "mnv2_expand_256x56x56x24to144": ("conv2d", lambda: cases.conv_case(seed=0, n=256, h=56, w=56, cin=24, cout=144, k=1, per_channel=True, out_scale=0.0235, out_zp=0), "hbm"),
        "mnv2_expand_256x28x28x32to192": ("conv2d", lambda: cases.conv_case(seed=0, n=256, h=28, w=28, cin=32, cout=192, k=1, per_channel=True, out_scale=0.0235, out_zp=0), "hbm"),
        "mnv2_expand_256x14x14x64to384": ("conv2d", lambda: cases.conv_case(seed=0, n=256, h=14, w=14, cin=64, cout=384, k=1, per_channel=True, out_scale=0.0235, out_zp=0), "hbm"),
        "mnv2_expand_256x14x14x96to576": ("conv2d", lambda: cases.conv_case(seed=0, n=256, h=14, w=14, cin=96, cout=576, k=1, per_channel=True, out_scale=0.0235, out_zp=0), "hbm"),
        "mnv2_expand_256x7x7x160to960": ("conv2d", lambda: cases.conv_case(seed=0, n=256, h=7, w=7, cin=160, cout=960, k=1, per_channel=True, out_scale=0.0235, out_zp=0), "hbm"),
        "mnv2_project_256x56x56x144to24": ("conv2d", lambda: cases.conv_case(seed=0, n=256, h=56, w=56, cin=144, cout=24, k=1, per_channel=True, out_scale=0.3, act=0, out_zp=128), "hbm"),
        "mnv2_project_256x112x112x32to16": ("conv2d", lambda: cases.conv_case(seed=0, n=256, h=112, w=112, cin=32, cout=16, k=1, per_channel=True, out_scale=0.3, act=0, out_zp=128), "hbm"),
        "mnv2_stem_256x224x224x3to32": ("conv2d", lambda: cases.conv_case(seed=0, n=256, h=224, w=224, cin=3, cout=32, k=3, stride=2, per_channel=True, out_scale=0.0235, out_zp=0), "hbm"),
        "mnv2_dw_256x56x56x144_s1": ("depthwise", lambda: cases.depthwise_case(seed=0, n=256, h=56, w=56, c=144, in_zp=0, out_scale=0.0235), "hbm"),
        "mnv2_dw_256x112x112x96_s2": ("depthwise", lambda: cases.depthwise_case(seed=0, n=256, h=112, w=112, c=96, stride=2, in_zp=0, out_scale=0.0235), "hbm"),
        "mnv2_add_256x56x56x24": ("add", None, "hbm"),
        "mnv2_pool_256x7x7x1280": ("avgpool", None, "hbm"),
    }


KERNEL_OF_IMPL = {0: "conv_direct_kernel", 1: "tc_gemm_kernel", 2: "gemv_kernel", 3: "dw3x3_ring_kernel", 4: "eltwise"}


def make_op(enn, ctx, cases, name):
    """Prepared operator + its host inputs for one named configuration."""
    kind, mk, bound = op_configs(cases)[name]
    if kind == "add":
        count = 256 * 56 * 56 * 24
        rng = np.random.default_rng(0)
        x = rng.integers(0, 256, count, dtype=np.int64).astype(np.uint8)
        x2 = rng.integers(0, 256, count, dtype=np.int64).astype(np.uint8)
        d = enn.AddDesc(count=count, activation=0, act_dtype=enn.U8, in0_scale=0.031, in0_zp=120, in1_scale=0.047, in1_zp=131,
                        out_scale=0.06, out_zp=126)
        return kind, bound, (d, x, x2), (lambda: enn.add(ctx, d))
    if kind == "avgpool":
        x = np.random.default_rng(0).integers(0, 256, (256, 7, 7, 1280), dtype=np.int64).astype(np.uint8)
        d = enn.PoolDesc(n=256, h=7, w=7, c=1280, kh=7, kw=7, stride_h=1, stride_w=1, pad_t=0, pad_l=0, out_h=1, out_w=1,
                         activation=0, act_dtype=enn.U8, out_scale=0.02, out_zp=0)
        return kind, bound, (d, x, None), (lambda: enn.avgpool(ctx, d))
    d, x, w, b, sc = mk()
    return kind, bound, (d, x, w, b, sc), (lambda: getattr(enn, kind)(ctx, d, w, b, sc))


def time_op(enn, ctx, cu, cases, name, reps=20, warmup=3):
    """Device-resident timing of one operator: `reps` back-to-back launches over rotating input/output
    buffer sets whose total size exceeds twice the L2, bracketed by CUDA events."""
    kind, bound, cfg, mk = make_op(enn, ctx, cases, name)
    x = cfg[1]
    x2 = cfg[2] if kind == "add" else None
    wbytes = cfg[2].nbytes if kind not in ("add", "avgpool") else 0
    op = mk()
    info = op.info
    # Operators whose traffic is mostly weights (FullyConnected) rotate over several prepared instances as well, so that
    # the weights of one launch have left the L2 before they are read again.
    nops = int(min(24, -(-(280 << 20) // wbytes))) if wbytes >= (4 << 20) else 1
    ops = [op] + [mk() for _ in range(nops - 1)]
    per_set = x.nbytes * (2 if x2 is not None else 1) + info.out_bytes
    nsets = int(max(2, min(64, -(-(280 << 20) // per_set))))
    xs = [ctx.to_device(x) for _ in range(nsets)]
    x2s = [ctx.to_device(x2) for _ in range(nsets)] if x2 is not None else None
    ys = [ctx.malloc(max(1, info.out_bytes)) for _ in range(nsets)]
    reps = max(reps, nops)

    def run(i):
        if x2s is not None:
            ops[i % nops].execute2(xs[i % nsets], x2s[i % nsets], ys[i % nsets])
        else:
            ops[i % nops].execute(xs[i % nsets], ys[i % nsets])

    for i in range(max(warmup, nops)):
        run(i)
    ctx.sync()
    e0, e1 = cu.event(), cu.event()
    cu.record(e0, ctx.stream)
    for i in range(reps):
        run(i)
    cu.record(e1, ctx.stream)
    ctx.sync()
    ms_eager = cu.elapsed_ms(e0, e1) / reps
    # The same `reps` launches captured once into a CUDA graph and replayed: operators of a few microseconds are bound by
    # the host's launch rate when every call comes from the Python loop above, and the graph shows the device's time.
    ms, timing = ms_eager, "eager launches"
    exe = cu.capture(ctx.stream, lambda: [run(i) for i in range(reps)])
    if exe is not None:
        cu.launch_graph(exe, ctx.stream)
        ctx.sync()
        cu.record(e0, ctx.stream)
        for _ in range(5):
            cu.launch_graph(exe, ctx.stream)
        cu.record(e1, ctx.stream)
        ctx.sync()
        ms_graph = cu.elapsed_ms(e0, e1) / (5 * reps)
        cu.destroy_graph(exe)
        if ms_graph < ms_eager:
            ms, timing = ms_graph, "CUDA graph of the same launches"
    for p in xs + ys + (x2s or []):
        ctx.free(p)
    res = dict(workload=name, impl=int(info.impl), bound=bound, ms=ms, launches_per_step=int(info.kernel_launches),
               tops=2 * info.macs / (ms * 1e-3) / 1e12, gbs=info.algorithmic_bytes / (ms * 1e-3) / 1e9,
               macs=int(info.macs), algorithmic_bytes=int(info.algorithmic_bytes), buffer_sets=nsets, weight_sets=nops, timing=timing,
               ms_eager=ms_eager)
    for o in ops:
        o.release()
    return res, (kind, cfg)


def cpu_baseline_op(kind, cfg, max_seconds=3.0):
    """The oracle's version of one operator on a bounded slice of its batch: (seconds per call, rows taken, rows)."""
    from oracle import orc
    orc.set_num_threads(host_threads())
    if kind == "add":
        d, x, x2 = cfg
        total = int(d.count)
        ns = min(total, 1 << 22)
        ds = type(d).from_buffer_copy(d)
        ds.count = ns
        fn = lambda: orc.add(ds, x[:ns], x2[:ns])
    elif kind == "avgpool":
        d, x, _ = cfg
        total, ns = d.n, min(d.n, 64)
        ds = type(d).from_buffer_copy(d)
        ds.n = ns
        xs = np.ascontiguousarray(x[:ns])
        fn = lambda: orc.avgpool(ds, xs)
    else:
        d, x, w, b, sc = cfg
        f = getattr(orc, kind)
        ds = type(d).from_buffer_copy(d)
        if kind == "fully_connected":
            ns, total = min(d.m, 64), d.m
            ds.m = ns
        else:
            ns, total = min(d.n, 8), d.n
            ds.n = ns
        xs = np.ascontiguousarray(x[:ns])
        fn = lambda: f(ds, xs, w, b, sc)
    fn()
    t0 = time.perf_counter()
    reps = 0
    while True:
        fn()
        reps += 1
        if time.perf_counter() - t0 > max_seconds or reps >= 20:
            break
    return (time.perf_counter() - t0) / reps, ns, total, reps


# ---------------------------------------------------------------------------------------------------
# MobileNetV2 graph
# ---------------------------------------------------------------------------------------------------
def kernel_of_layer(L, impl):
    if L["kind"] == "conv" and L["cin"] == 3:
        return "conv3x3c3_kernel"
    if L["kind"] == "add":
        return "add_kernel_lut2"
    if L["kind"] == "pool":
        return "avgpool_vec4_kernel"
    return KERNEL_OF_IMPL.get(impl, "other")


class Lane:
    """One operator list with its own context (stream), buffers, CUDA graph and pinned host buffers."""

    def __init__(self, enn, mn, device, layers, batch, x, out_bytes, options=()):
        self.enn = enn
        self.ctx = enn.Context(device)
        for name, value in options:
            self.ctx.set_option(name, value)
        self.ol, self.info = mn.make_oplist(enn, self.ctx, layers, batch)
        self.ctx.upload(self.ol.tensor_ptr(self.info["tensor_ids"]["input"]), x)
        self.host = []
        for _ in range(2):
            hin, hout = C.c_void_p(), C.c_void_p()
            assert enn.lib.enn_b200_host_alloc(x.nbytes, C.byref(hin)) == 0
            assert enn.lib.enn_b200_host_alloc(out_bytes, C.byref(hout)) == 0
            C.memmove(hin, x.ctypes.data, x.nbytes)
            self.host.append((hin.value, hout.value))
        self.out_bytes = out_bytes
        self.n = 0

    def submit(self):
        hin, hout = self.host[self.n & 1]
        self.ol.submit_host_ptrs([hin], [hout])
        self.n += 1
        return hout

    def logits(self, which):
        return np.ctypeslib.as_array((C.c_uint8 * self.out_bytes).from_address(self.host[which][1])).copy()


class DevView:
    """Zero-copy view of device bytes for torch (CUDA array interface)."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (int(ptr), False), "version": 2}


def run_mobilenet(args, enn, cu, cases, rank, world, local, barrier, torch, dist):
    mn = importlib.import_module("cl_eden_kernel_b200.mobilenet")
    layers, _ = mn.build_model(seed=0, calib_images=1)
    if GLOBAL_BATCH % world:
        raise SystemExit(f"the {GLOBAL_BATCH}-image batch does not split over {world} GPUs")
    per_rank = GLOBAL_BATCH // world
    x_full = np.random.default_rng(1000).integers(0, 256, (GLOBAL_BATCH, 224, 224, 3), dtype=np.int64).astype(np.uint8)
    x = np.ascontiguousarray(x_full[rank * per_rank:(rank + 1) * per_rank])
    classes = layers[-1]["cout"]
    out_bytes = per_rank * classes
    multi = world > 1

    # ---- lanes: how many operator lists share this GPU, and the share of its SMs each list's kernels may take.
    # Default: up to twelve lists whose persistent kernels launch at most a quarter of the SMs (option grid_cap), so that
    # four kernels of different steps run side by side; "auto" times 4, 8, 10 and 12 lists on the step count that will
    # be timed and keeps the best.
    max_lanes = args.lanes if args.lanes > 0 else 12
    sm_count = torch.cuda.get_device_properties(local).multi_processor_count
    grid_cap = args.grid_cap if args.grid_cap >= 0 else (sm_count // 4 if max_lanes >= 4 else 0)
    user_options = [(kv.split("=")[0], int(kv.split("=")[1])) for kv in args.opt]
    options = user_options + ([("grid_cap", grid_cap)] if grid_cap > 0 else [])
    lanes = [Lane(enn, mn, local, layers, per_rank, x, out_bytes, options) for _ in range(max_lanes)]
    info = lanes[0].info
    stats = lanes[0].ol.stats()

    def device_steps(use, steps):
        """`steps` graph launches handed to the first `use` lanes in turn; device time between the first launch and
        the completion of the last, measured on lane 0's stream."""
        e0, e1 = cu.event(), cu.event()
        tails = [cu.event() for _ in range(use)]
        for l in lanes[:use]:
            l.ctx.sync()
        cu.record(e0, lanes[0].ctx.stream)
        for i in range(steps):
            lanes[i % use].ol.execute_device()
        for k in range(1, use):
            cu.record(tails[k], lanes[k].ctx.stream)
            cu.stream_wait(lanes[0].ctx.stream, tails[k])
        cu.record(e1, lanes[0].ctx.stream)
        return cu.elapsed_ms(e0, e1)

    # The clock sampler starts here, well ahead of the timed regions, so that the start-up of nvidia-smi does not fall
    # into them; the samples from `mark()` on are the ones summarised.
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        sampler.wait_first_sample()
    for l in lanes:
        for _ in range(args.warmup):
            l.ol.execute_device()
        l.ctx.sync()
    if args.lanes > 0:
        use = args.lanes
        lane_trials = None
    else:
        lane_trials = {}
        for s in (4, 8, 10, 12):      # on the step count that will be timed: a K that divides by the lanes leaves no partial round
            device_steps(s, 2 * s)
            lane_trials[s] = device_steps(s, args.steps) / args.steps
        if multi:      # every rank must make the same choice: take rank 0's
            t = torch.tensor([lane_trials[s] for s in sorted(lane_trials)], device="cuda", dtype=torch.float64)
            dist.broadcast(t, 0)
            lane_trials = {s: v for s, v in zip(sorted(lane_trials), t.tolist())}
        use = min(lane_trials, key=lane_trials.get)

    # Last warm-up pass on the lanes that will be timed, after everything else that precedes the timed region (the lane
    # trial and, at N > 1, the first collective of the run, whose set-up otherwise slows the next pass by up to 9 %).
    device_steps(use, 2 * use)

    # No collector pause inside the timed regions: a generation-2 collection of this process takes milliseconds, which is
    # a third of a 20-step region at 2 GPUs (and whether it falls inside depends on how many objects were made before).
    gc.collect()
    gc.disable()

    # ---- device-resident: K graph launches between two events ----
    sampler.mark()
    barrier()
    total_ms = device_steps(use, args.steps)
    barrier()

    # ---- end to end: host buffers (pinned) through enn_b200_oplist_submit / _wait, logits gathered on rank 0 ----
    # Every step copies its images host->device and its logits device->host (the copy-in of a step overlaps the
    # operators of the step before); at N > 1 every step's logits also travel to rank 0 (NCCL gather of the device
    # copy after the lane's graph, then device->host there).  The region ends when the last result has landed.
    ext, src_views, gath, gath_host, gath_rows, gstream, gdone = None, {}, None, None, None, None, {}
    if multi:
        ext = [torch.cuda.ExternalStream(l.ctx.stream.value if hasattr(l.ctx.stream, "value") else int(l.ctx.stream)) for l in lanes[:use]]
        # The gathers run on a stream of their own per lane: a lane's next graph does not wait for the other ranks, only
        # the graph that will overwrite the gathered output buffer (two submissions later) does.
        gstream = [torch.cuda.Stream() for _ in lanes[:use]]
        if rank == 0:
            gath = [torch.empty((world, out_bytes), dtype=torch.uint8, device="cuda") for _ in range(use)]
            gath_host = [torch.empty((world, out_bytes), dtype=torch.uint8).pin_memory() for _ in range(use)]
            gath_rows = [list(g.unbind(0)) for g in gath]

    # Lanes that share the GPU by SM shares are submitted in rounds (enn_b200_oplist_submit_round): the lanes of a round
    # fill the GPU together and start together, the next round's inputs travel meanwhile.
    # The end-to-end leg of a short run uses the lanes of one round only: all lanes (two rounds in flight at once) gain
    # 3 % on long runs (160 steps: 199 k against 194 k images/s) and lose 5 % on a 20-step run, which starts from an empty
    # pipeline (168 k against 177 k).
    round_size = max(1, min(use, sm_count // grid_cap)) if grid_cap > 0 else 1
    use_dev = use
    if grid_cap > 0:
        if args.e2e_lanes > 0:
            use = max(round_size, min(use, args.e2e_lanes))
        elif args.steps < 16 * round_size:
            use = round_size

    def e2e_steps(steps):
        i = 0
        while i < steps:
            first = i % use
            ks = [(first + j) % use for j in range(min(round_size, steps - i))]
            if multi:
                for k in ks:      # the output buffer this submission writes: its last gather must have read it
                    ev = gdone.get((k, lanes[k].n & 1))
                    if ev is not None:
                        ext[k].wait_event(ev)
            if len(ks) == 1:
                lanes[ks[0]].submit()
            else:
                bufs = [lanes[k].host[lanes[k].n & 1] for k in ks]
                enn.OpList.submit_round([lanes[k].ol for k in ks], [[b[0]] for b in bufs], [[b[1]] for b in bufs])
                for k in ks:
                    lanes[k].n += 1
            for k in ks:
                if multi:
                    ptr = lanes[k].ol.last_output_ptr(0).value
                    src = src_views.get(ptr)        # a list alternates between two output buffers: wrap each once
                    if src is None:
                        src = src_views[ptr] = torch.as_tensor(DevView(ptr, out_bytes), device="cuda")
                    ready = torch.cuda.Event()
                    ready.record(ext[k])
                    with torch.cuda.stream(gstream[k]):
                        gstream[k].wait_event(ready)
                        dist.gather(src, gath_rows[k] if rank == 0 else None, dst=0)
                        if rank == 0:
                            gath_host[k].copy_(gath[k], non_blocking=True)
                        done = torch.cuda.Event()
                        done.record(gstream[k])
                    gdone[(k, (lanes[k].n - 1) & 1)] = done
            i += len(ks)
        for l in lanes[:use]:
            l.ol.wait()
        if multi:
            for g in gstream:
                g.synchronize()

    e2e_steps(2 * use)
    barrier()
    t0, t1 = cu.event(), cu.event()
    tails = [cu.event() for _ in range(use)]
    cu.record(t0, lanes[0].ctx.stream)
    e2e_steps(args.steps)
    for k in range(1, use):
        cu.record(tails[k], lanes[k].ctx.stream)
        cu.stream_wait(lanes[0].ctx.stream, tails[k])
    cu.record(t1, lanes[0].ctx.stream)
    barrier()
    e2e_ms = cu.elapsed_ms(t0, t1)
    gc.enable()
    clocks = sampler.stop() if rank == 0 else None
    logits = lanes[0].logits(1 if (lanes[0].n & 1) == 0 else 0).reshape(per_rank, classes)   # the buffer of lane 0's latest step
    gathered = gath_host[0].numpy().reshape(GLOBAL_BATCH, classes).copy() if multi and rank == 0 else None

    # ---- per-layer timing (rank 0): which kernel dominates, and its achieved bandwidth ----
    # Two timings per layer: launched on every lane at once (the regime of the timed region: each launch on its share
    # of the SMs, four side by side; a single launch cannot be timed there, the elapsed time over the launches can),
    # and one launch at a time with the whole GPU (a context without the share).
    per_kernel = {}
    if rank == 0:
        alone = enn.Context(local)
        for name, value in user_options:
            alone.set_option(name, value)
        shared = lanes[:use_dev] if grid_cap > 0 and use_dev > 1 else []

        def make_op(ctx, L, d):
            if L["kind"] == "conv":
                return enn.conv2d(ctx, d, L["w"], L["bias"], L["scales"])
            if L["kind"] == "dw":
                return enn.depthwise(ctx, d, L["w"], L["bias"], L["scales"])
            if L["kind"] == "fc":
                return enn.fully_connected(ctx, d, L["w"].reshape(L["cout"], L["cin"]), L["bias"], L["scales"])
            if L["kind"] == "add":
                return enn.add(ctx, d)
            return enn.avgpool(ctx, d)

        def runner(op, lane, L):
            # fresh operator handles on a list's own buffers (graph nodes are owned by the list)
            tid, ol = lane.info["tensor_ids"], lane.ol
            a, o = ol.tensor_ptr(tid[L["src"]]), ol.tensor_ptr(tid[L["name"]])
            if L["kind"] == "add":
                b2 = ol.tensor_ptr(tid[L["src2"]])
                return lambda: op.execute2(a, b2, o)
            return lambda: op.execute(a, o)

        for L, pl in zip(layers, info["per_layer"]):
            d = mn.layer_descs(enn, L, per_rank)
            # (1) alone: the whole GPU to one launch at a time
            op = make_op(alone, L, d)
            run = runner(op, lanes[0], L)
            run()
            ea, eb = cu.event(), cu.event()
            cu.record(ea, alone.stream)
            for _ in range(5):
                run()
            cu.record(eb, alone.stream)
            alone.sync()
            ms_alone = cu.elapsed_ms(ea, eb) / 5
            op.release()
            # (2) as in the timed region: the same layer on every lane at once, each launch on its share of the SMs
            ms_shared = None
            if shared:
                ops = [make_op(l.ctx, L, d) for l in shared]
                runs = [runner(op_k, l, L) for op_k, l in zip(ops, shared)]
                for r in runs:
                    r()
                for l in shared:
                    l.ctx.sync()
                ea, eb = cu.event(), cu.event()
                tails = [cu.event() for _ in shared]
                cu.record(ea, shared[0].ctx.stream)
                for _ in range(5):
                    for r in runs:
                        r()
                for k in range(1, len(shared)):
                    cu.record(tails[k], shared[k].ctx.stream)
                    cu.stream_wait(shared[0].ctx.stream, tails[k])
                cu.record(eb, shared[0].ctx.stream)
                for l in shared:
                    l.ctx.sync()
                ms_shared = cu.elapsed_ms(ea, eb) / (5 * len(shared))
                for op_k in ops:
                    op_k.release()
            k = kernel_of_layer(L, pl["impl"])
            acc = per_kernel.setdefault(k, dict(ms=0.0, ms_alone=0.0, bytes=0, macs=0, launches=0))
            acc["ms"] += ms_shared if ms_shared is not None else ms_alone
            acc["ms_alone"] += ms_alone
            acc["bytes"] += pl["bytes"]
            acc["macs"] += pl["macs"]
            acc["launches"] += pl["launches"]
        alone.close()
    ol_info = dict(macs=info["macs"], bytes=info["bytes"], launches=info["launches"], stats=stats, layers=len(layers))
    return dict(total_ms=total_ms, e2e_ms=e2e_ms, clocks=clocks, per_rank=per_rank, h2d=int(x.nbytes), d2h=int(out_bytes),
                per_kernel=per_kernel, info=ol_info, logits=logits, gathered=gathered, layers=layers, x=x, x_full=x_full,
                lanes=use_dev, lane_trials=lane_trials, mn=mn, lane_objs=lanes, grid_cap=grid_cap, round_size=round_size, e2e_lanes=use)


def cpu_baseline_mobilenet(layers, x, max_images=8):
    """The oracle graph timed on the host cores over a bounded sample of the batch; also returns its logits."""
    from oracle import mobilenet_ref, orc
    orc.set_num_threads(host_threads())
    types, mn = load_plain("abi_types"), load_plain("mobilenet")
    xs = np.ascontiguousarray(x[:max_images])
    y = mobilenet_ref.run_oracle(layers, xs, types=types, mobilenet=mn)
    t0 = time.perf_counter()
    reps = 0
    while True:
        mobilenet_ref.run_oracle(layers, xs, types=types, mobilenet=mn)
        reps += 1
        if time.perf_counter() - t0 > 8.0 or reps >= 10:
            break
    dt = (time.perf_counter() - t0) / reps
    return {"value": len(xs) / dt, "unit": "images/s", "cores": orc.num_threads(), "kind": "port",
            "sample": f"{len(xs)} of {x.shape[0]} images of the same MobileNetV2-u8 graph, {reps} repetitions, {dt * 1e3:.0f} ms each"}, y


def graph_config(mn, layers, world):
    """The `config` object of the default workload; the same for both arms."""
    per_rank = GLOBAL_BATCH // max(1, world)
    macs, nbytes = mn.graph_work(layers, GLOBAL_BATCH)
    return {"workload": WORKLOAD_TEXT, "global_batch": GLOBAL_BATCH, "images_per_gpu": per_rank,
            "l2": "no flush needed: the activations a step streams (several hundred MB per GPU) exceed the 126 MB L2",
            "sharding": f"contiguous slices of {per_rank} images per rank; no collective on the data path; the {GLOBAL_BATCH} x 1000 logits are gathered on rank 0",
            "ops_per_step": len(layers), "gmacs_per_step": macs / 1e9, "algorithmic_gbytes_per_step": nbytes / 1e9}


def run_ours(args):
    import torch
    import torch.distributed as dist
    enn = load_package()
    cases = importlib.import_module("cl_eden_kernel_b200.workloads")
    rank, world, local = dist_env()
    if world > 1 and args.gpus != world:
        raise SystemExit("--gpus must equal WORLD_SIZE under torchrun")
    multi = world > 1
    torch.cuda.set_device(local)
    if multi:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = enn.Context(local)
    options = [(kv.split("=")[0], int(kv.split("=")[1])) for kv in args.opt]      # planner / tuning switches (none changes a result)
    for name, value in options:
        ctx.set_option(name, value)
    cu = Cuda()

    def barrier():
        ctx.sync()
        torch.cuda.synchronize()
        if multi:
            dist.barrier()
        ctx.sync()

    peaks = measured_peaks()
    result = None
    if args.workload == DEFAULT_WORKLOAD:
        r = run_mobilenet(args, enn, cu, cases, rank, world, local, barrier, torch, dist)
        total_ms, e2e_ms = r["total_ms"], r["e2e_ms"]
        by_rank = e2e_by_rank = None
        if multi:
            t = torch.tensor([total_ms, e2e_ms], device="cuda", dtype=torch.float64)
            every = [torch.zeros_like(t) for _ in range(world)]
            dist.all_gather(every, t)
            by_rank = [round(v[0].item() / args.steps, 4) for v in every]
            e2e_by_rank = [round(v[1].item() / args.steps, 4) for v in every]
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            total_ms, e2e_ms = t.tolist()
        if rank == 0:
            units = GLOBAL_BATCH * args.steps
            pk = r["per_kernel"]
            dom = max(pk, key=lambda k: pk[k]["ms"]) if pk else None
            roof = None
            if dom:
                launches = max(1, pk[dom]["launches"])
                avg_ms = pk[dom]["ms"] / launches
                ach = pk[dom]["bytes"] / (pk[dom]["ms"] * 1e-3) / 1e9
                ratio = NCU_TRAFFIC_RATIO.get(dom)
                roof = {"bound": "hbm", "kernel": dom, "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                        "frac": ach / peaks["hbm_gbs"],
                        "traffic": pk[dom]["bytes"] / launches * ratio if ratio else None,
                        "algorithmic_bytes_per_launch": pk[dom]["bytes"] / launches,
                        "peak_source": peaks["source"],
                        "avg_launch_ms": avg_ms, "launches_per_step": launches,
                        "share_of_step": pk[dom]["ms"] / sum(v["ms"] for v in pk.values()),
                        "timed": ("every layer launched on all %d lanes at once, as in the timed region (each launch on its share of "
                                  "%d SMs, four side by side), CUDA events around 5 such rounds; avg_launch_ms = elapsed / launches. "
                                  "per_kernel_ms_alone: one launch at a time with all SMs" % (r["lanes"], r["grid_cap"]))
                                 if r["grid_cap"] > 0 and r["lanes"] > 1 else "every layer launched alone, CUDA events, 5 launches each",
                        "per_kernel_ms_alone": {k: round(v["ms_alone"], 4) for k, v in pk.items()},
                        "per_kernel_frac_of_hbm_alone": {k: round(v["bytes"] / (v["ms_alone"] * 1e-3) / 1e9 / peaks["hbm_gbs"], 3) for k, v in pk.items()},
                        "whole_step": {"algorithmic_gbytes": r["info"]["bytes"] * world / 1e9,
                                       "achieved": r["info"]["bytes"] * world / (total_ms / args.steps * 1e-3) / 1e9 / world,
                                       "unit": "GB/s per GPU",
                                       "frac": r["info"]["bytes"] / (total_ms / args.steps * 1e-3) / 1e9 / peaks["hbm_gbs"]},
                        "per_kernel_ms": {k: round(v["ms"], 4) for k, v in pk.items()},
                        "per_kernel_frac_of_hbm": {k: round(v["bytes"] / (v["ms"] * 1e-3) / 1e9 / peaks["hbm_gbs"], 3) for k, v in pk.items()}}
            result = {
                "metric": "mobilenetv2_u8_images_per_s", "value": units / (total_ms * 1e-3), "unit": "images/s",
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms / args.steps,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
                "config": graph_config(r["mn"], r["layers"], world),
                "roofline": roof,
                "e2e": {"value": units / (e2e_ms * 1e-3), "unit": "images/s", "h2d_bytes_per_step": r["h2d"] * world,
                        "d2h_bytes_per_step": r["d2h"] * world},
                "gpu_launches": int(r["info"]["stats"]["kernel_launches"] * args.steps * world),      # the lists' own count (fused adds are one launch)
                "clocks": r["clocks"],
                "logits_checksum": int(r["logits"].astype(np.int64).sum()),
            }
            if by_rank:
                result["ms_per_step_by_rank"] = by_rank      # `ms_per_step` is their maximum
                result["e2e"]["ms_per_step_by_rank"] = e2e_by_rank
            result["lanes_per_gpu"] = r["lanes"]
            result["sm_share_per_lane"] = r["grid_cap"] if r["grid_cap"] > 0 else "all"
            result["e2e"]["lanes"] = r["e2e_lanes"]
            result["e2e"]["lanes_per_round"] = r["round_size"]
            result["device_bytes_per_lane"] = r["info"]["stats"]["device_bytes"]
            if r["lane_trials"]:
                result["lane_trial_ms_per_step"] = {str(k): round(v, 4) for k, v in r["lane_trials"].items()}
            if multi:
                # The gathered logits of the partitioned run against the same 256 images on this GPU alone.
                lane = Lane(enn, r["mn"], local, r["layers"], GLOBAL_BATCH, r["x_full"], GLOBAL_BATCH * r["layers"][-1]["cout"])
                lane.submit()
                lane.ol.wait()
                full = lane.logits(0).reshape(GLOBAL_BATCH, -1)
                if not np.array_equal(full, r["gathered"]):
                    raise SystemExit("gathered logits of the partitioned batch differ from the single-GPU result")
                result["gathered_equals_single_gpu"] = True
                lane.ol.destroy()
            if world == 1 and not args.skip_cpu_baseline:
                result["cpu_baseline"], y_ref = cpu_baseline_mobilenet(r["layers"], r["x"])
                if not np.array_equal(r["logits"][:len(y_ref)], y_ref.reshape(len(y_ref), -1)):
                    raise SystemExit("logits of the timed graph differ from the CPU oracle")
                result["parity_checked_images"] = int(len(y_ref))
            if world == 1 and not args.skip_per_op:
                per_op = []
                i8_peak = ctx.mma_peak(2, 256, 16384)      # kind::i8 on pseudo-random operand bytes
                for name in op_configs(cases):
                    if name.startswith("mnv2_"):
                        continue
                    res, (kind, cfg) = time_op(enn, ctx, cu, cases, name)
                    res["frac_of_hbm_measured"] = res["gbs"] / peaks["hbm_gbs"]
                    res["frac_of_int8_tensor_measured"] = res["tops"] / i8_peak
                    res["frac_of_int8_tensor_nominal_4500"] = res["tops"] / 4500.0
                    if not args.skip_cpu_baseline:
                        dt, ns, total, reps = cpu_baseline_op(kind, cfg, max_seconds=1.5)
                        res["cpu_baseline"] = {"ms_full_op_extrapolated": dt * 1e3 * total / ns, "cores": host_threads(), "kind": "port",
                                               "sample": f"{ns} of {total} batch rows, {reps} repetitions, {dt * 1e3:.1f} ms each"}
                    per_op.append(res)
                result["per_op"] = per_op
                result["int8_tensor_peak_measured_tops"] = i8_peak
                result["int8_tensor_peak_zero_operands_tops"] = ctx.mma_peak(0, 256, 16384)
    else:
        res, (kind, cfg) = time_op(enn, ctx, cu, cases, args.workload, reps=args.steps, warmup=args.warmup)
        # end to end: one operator through upload / execute / download with pinned host buffers
        _, _, _, mk = make_op(enn, ctx, cases, args.workload)
        op = mk()
        info = op.info
        x = cfg[1]
        x2 = cfg[2] if kind == "add" else None
        hin, hin2, hout = C.c_void_p(), C.c_void_p(), C.c_void_p()
        enn.lib.enn_b200_host_alloc(x.nbytes, C.byref(hin))
        enn.lib.enn_b200_host_alloc(x.nbytes, C.byref(hin2))
        enn.lib.enn_b200_host_alloc(max(1, info.out_bytes), C.byref(hout))
        C.memmove(hin, x.ctypes.data, x.nbytes)
        if x2 is not None:
            C.memmove(hin2, x2.ctypes.data, x2.nbytes)
        xd, x2d, yd = ctx.malloc(x.nbytes), ctx.malloc(x.nbytes), ctx.malloc(max(1, info.out_bytes))
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()

        def e2e_once():
            enn.lib.enn_b200_upload(ctx.h, xd, hin, x.nbytes)
            if x2 is not None:
                enn.lib.enn_b200_upload(ctx.h, x2d, hin2, x.nbytes)
                op.execute2(xd, x2d, yd)
            else:
                op.execute(xd, yd)
            enn.lib.enn_b200_download(ctx.h, hout, yd, info.out_bytes)

        for _ in range(2):
            e2e_once()
        barrier()
        e0, e1 = cu.event(), cu.event()
        cu.record(e0, ctx.stream)
        for _ in range(args.steps):
            e2e_once()
        cu.record(e1, ctx.stream)
        barrier()
        e2e_ms = cu.elapsed_ms(e0, e1) / args.steps
        clocks = sampler.stop() if rank == 0 else None
        ms = res["ms"]
        if multi:
            t = torch.tensor([ms, e2e_ms], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms, e2e_ms = t.tolist()
        if rank == 0:
            hbm = res["bound"] == "hbm"
            unit = "GB/s" if hbm else "TOP/s"
            per_step = res["algorithmic_bytes"] / 1e9 if hbm else 2 * res["macs"] / 1e12
            i8_peak = ctx.mma_peak(2, 256, 16384)      # kind::i8 on pseudo-random operand bytes
            peak = peaks["hbm_gbs"] if hbm else i8_peak
            ach = per_step / (res["ms"] * 1e-3)
            kname = {"depthwise": "dw3x3_ring_kernel", "add": "add_kernel_lut2", "avgpool": "avgpool_vec4_kernel"}.get(kind, KERNEL_OF_IMPL.get(res["impl"]))
            result = {
                "metric": ("hbm_gbs_" if hbm else "int8_tops_") + args.workload, "value": world * per_step / (ms * 1e-3),
                "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
                "config": {"workload": args.workload, "l2": f"{res['buffer_sets']} rotating input/output buffer sets, together larger than twice the L2",
                           "sharding": "independent replicas per rank, no collective"},
                "roofline": {"bound": "hbm" if hbm else "tensor", "kernel": kname, "achieved": ach, "peak": peak,
                             "unit": unit, "frac": ach / peak, "traffic": None,
                             "peak_source": peaks["source"] if hbm else "measured tcgen05.mma kind::i8 rate on random operand bytes (enn_b200_measure_mma_peak)",
                             "frac_of_nominal_4500_tops": None if hbm else ach / 4500.0},
                "e2e": {"value": world * per_step / (e2e_ms * 1e-3), "unit": unit, "h2d_bytes_per_step": int(x.nbytes * (2 if x2 is not None else 1)),
                        "d2h_bytes_per_step": int(info.out_bytes)},
                "gpu_launches": int(res["launches_per_step"] * args.steps),
                "clocks": clocks,
            }
            if world == 1 and not args.skip_cpu_baseline:
                dt, ns, total, reps = cpu_baseline_op(kind, cfg, max_seconds=8.0)
                frac = ns / total
                result["cpu_baseline"] = {"value": per_step * frac / dt, "unit": unit, "cores": host_threads(), "kind": "port",
                                          "sample": f"{ns} of {total} batch rows of {args.workload}, {reps} repetitions, {dt * 1e3:.1f} ms each"}
    if rank == 0 and result is not None:
        print(json.dumps(result), flush=True)
    if multi:
        dist.destroy_process_group()


def run_reference(args):
    """The CPU oracle on the host cores: K steps, each a bounded sample of the workload.  Loads the descriptors, the
    workload generators and the oracle only; the CUDA library is not touched."""
    rank, world, _ = dist_env()
    if rank != 0:
        return
    from oracle import mobilenet_ref, orc
    orc.set_num_threads(host_threads())          # a launcher may have set OMP_NUM_THREADS=1 for its ranks
    types, cases = load_plain("abi_types"), load_plain("workloads")
    if args.workload == DEFAULT_WORKLOAD:
        mn = load_plain("mobilenet")
        layers, _ = mn.build_model(seed=0, calib_images=1)
        n = 8
        x = np.random.default_rng(1000).integers(0, 256, (n, 224, 224, 3), dtype=np.int64).astype(np.uint8)
        for _ in range(args.warmup):
            mobilenet_ref.run_oracle(layers, x[:2], types=types, mobilenet=mn)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            mobilenet_ref.run_oracle(layers, x, types=types, mobilenet=mn)
        dt = (time.perf_counter() - t0) / args.steps
        v, unit, metric = n / dt, "images/s", "mobilenetv2_u8_images_per_s"
        sample = f"each step = the first {n} images of the {GLOBAL_BATCH}-image batch through the CPU oracle graph"
        cfg = graph_config(mn, layers, args.gpus)
        scaling = "strong"
    else:
        kind, mk, bound = op_configs(cases)[args.workload]
        if mk is None:
            print(json.dumps({"impl": "reference", "unavailable": "this profiling workload has no CPU arm"}), flush=True)
            return
        d, x, w, b, sc = mk()
        dt, ns, total, reps = cpu_baseline_op(kind, (d, x, w, b, sc), max_seconds=3.0)
        hbm = bound == "hbm"
        if kind == "fully_connected":
            macs, abytes = d.m * d.k * d.n, d.m * d.k + d.k * d.n + d.m * d.n + 12 * d.n
        else:
            abytes = x.nbytes + w.nbytes + 12 * d.cout
            macs = 0
        per_step = (abytes / 1e9 if hbm else 2 * macs / 1e12) * ns / total
        v, unit, metric = per_step / dt, ("GB/s" if hbm else "TOP/s"), ("hbm_gbs_" if hbm else "int8_tops_") + args.workload
        sample = f"{ns} of {total} batch rows"
        cfg = {"workload": args.workload}
        scaling = "weak"
    print(json.dumps({
        "impl": "reference", "metric": metric, "value": v, "unit": unit, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
        "dtype": "u8", "data": "synthetic", "config": cfg,
        "cpu_baseline": {"value": v, "unit": unit, "cores": orc.num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD)
    ap.add_argument("--lanes", type=int, default=0, help="operator lists per GPU that take the steps in turn (0: time 4, 8, 10 and 12 and keep the best)")
    ap.add_argument("--e2e-lanes", type=int, default=0, help="lanes of the end-to-end leg (0: the lanes of one round for runs under 64 steps, else all)")
    ap.add_argument("--grid-cap", type=int, default=-1, help="SMs a lane's persistent kernels may occupy (-1: a quarter of the GPU with four or more lanes; 0: all)")
    ap.add_argument("--opt", action="append", default=[], metavar="NAME=VALUE", help="library option for every context (tuning runs), e.g. no_fuse=1")
    ap.add_argument("--skip-cpu-baseline", action="store_true", help="omit the CPU leg (profiling runs)")
    ap.add_argument("--skip-per-op", action="store_true", help="omit the single-operator table (profiling runs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
