"""ctypes binding of libenn_b200.so, the C ABI over the sm_100a quantized-operator kernels.

This module is plumbing for tests, the benchmark and Python callers: every operator call goes through the
same `extern "C"` entry points (include/enn_b200.h) that a C++ userdriver binds.  There is no CPU
fallback: if the shared library is missing, import fails; if no CUDA device is present, creating a
`Context` fails.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libenn_b200.so")

try:
    from .abi_types import *          # noqa: F401,F403  (constants, descriptors, conv_desc)
    from .abi_types import ConvDesc, FcDesc, AddDesc, PoolDesc, OpInfo, MeanDesc, ConcatDesc, SoftmaxDesc, ResizeDesc
except ImportError:                   # loaded as a plain module
    from abi_types import *           # noqa: F401,F403
    from abi_types import ConvDesc, FcDesc, AddDesc, PoolDesc, OpInfo, MeanDesc, ConcatDesc, SoftmaxDesc, ResizeDesc

# Every symbol include/enn_b200.h declares, with its prototype: (restype, argtypes).
_P = C.c_void_p
PROTOTYPES = {
    "enn_b200_context_create": (C.c_int32, [C.c_int32, C.POINTER(_P)]),
    "enn_b200_context_destroy": (C.c_int32, [_P]),
    "enn_b200_malloc": (C.c_int32, [_P, C.c_size_t, C.POINTER(_P)]),
    "enn_b200_free": (C.c_int32, [_P, _P]),
    "enn_b200_upload": (C.c_int32, [_P, _P, _P, C.c_size_t]),
    "enn_b200_download": (C.c_int32, [_P, _P, _P, C.c_size_t]),
    "enn_b200_copy_device": (C.c_int32, [_P, _P, _P, C.c_size_t]),
    "enn_b200_stream_sync": (C.c_int32, [_P]),
    "enn_b200_host_alloc": (C.c_int32, [C.c_size_t, C.POINTER(_P)]),
    "enn_b200_host_free": (C.c_int32, [_P]),
    "enn_b200_last_error": (C.c_int32, [_P, C.c_char_p, C.c_size_t]),
    "enn_b200_stream": (_P, [_P]),
    "enn_b200_context_set_option": (C.c_int32, [_P, C.c_char_p, C.c_int32]),
    "enn_b200_conv2d_prepare": (C.c_int32, [_P, C.POINTER(ConvDesc), _P, _P, _P, C.POINTER(_P)]),
    "enn_b200_depthwise_prepare": (C.c_int32, [_P, C.POINTER(ConvDesc), _P, _P, _P, C.POINTER(_P)]),
    "enn_b200_deconv_prepare": (C.c_int32, [_P, C.POINTER(ConvDesc), _P, _P, _P, C.POINTER(_P)]),
    "enn_b200_fc_prepare": (C.c_int32, [_P, C.POINTER(FcDesc), _P, _P, _P, C.POINTER(_P)]),
    "enn_b200_add_prepare": (C.c_int32, [_P, C.POINTER(AddDesc), C.POINTER(_P)]),
    "enn_b200_avgpool_prepare": (C.c_int32, [_P, C.POINTER(PoolDesc), C.POINTER(_P)]),
    "enn_b200_maxpool_prepare": (C.c_int32, [_P, C.POINTER(PoolDesc), C.POINTER(_P)]),
    "enn_b200_mean_prepare": (C.c_int32, [_P, C.POINTER(MeanDesc), C.POINTER(_P)]),
    "enn_b200_concat_prepare": (C.c_int32, [_P, C.POINTER(ConcatDesc), C.POINTER(_P)]),
    "enn_b200_softmax_prepare": (C.c_int32, [_P, C.POINTER(SoftmaxDesc), C.POINTER(_P)]),
    "enn_b200_resize_bilinear_prepare": (C.c_int32, [_P, C.POINTER(ResizeDesc), C.POINTER(_P)]),
    "enn_b200_op_set_impl": (C.c_int32, [_P, C.c_int32]),
    "enn_b200_op_execute": (C.c_int32, [_P, _P, _P]),
    "enn_b200_op_execute2": (C.c_int32, [_P, _P, _P, _P]),
    "enn_b200_op_execute_n": (C.c_int32, [_P, C.POINTER(_P), C.c_int32, _P]),
    "enn_b200_op_execute_noalloc": (C.c_int32, [_P, _P, _P]),
    "enn_b200_op_rebind_constants": (C.c_int32, [_P, _P, _P]),
    "enn_b200_op_fuse_add": (C.c_int32, [_P, _P, C.c_int32]),
    "enn_b200_op_info": (C.c_int32, [_P, C.POINTER(OpInfo)]),
    "enn_b200_op_test_starve_next": (C.c_int32, [_P]),
    "enn_b200_op_clear_error": (C.c_int32, [_P]),
    "enn_b200_op_release": (C.c_int32, [_P]),
    "enn_b200_oplist_create": (C.c_int32, [_P, C.POINTER(_P)]),
    "enn_b200_oplist_add_tensor": (C.c_int32, [_P, C.c_int64, C.POINTER(C.c_int32)]),
    "enn_b200_oplist_add_op": (C.c_int32, [_P, _P, C.POINTER(C.c_int32), C.c_int32, C.c_int32]),
    "enn_b200_oplist_set_io": (C.c_int32, [_P, C.POINTER(C.c_int32), C.c_int32, C.POINTER(C.c_int32), C.c_int32]),
    "enn_b200_oplist_finalize": (C.c_int32, [_P]),
    "enn_b200_oplist_execute": (C.c_int32, [_P, C.POINTER(_P), C.POINTER(_P)]),
    "enn_b200_oplist_execute_device": (C.c_int32, [_P]),
    "enn_b200_oplist_submit": (C.c_int32, [_P, C.POINTER(_P), C.POINTER(_P)]),
    "enn_b200_oplist_submit_round": (C.c_int32, [C.POINTER(_P), C.c_int32, C.POINTER(C.POINTER(_P)), C.POINTER(C.POINTER(_P))]),
    "enn_b200_oplist_wait": (C.c_int32, [_P]),
    "enn_b200_oplist_tensor_ptr": (C.c_int32, [_P, C.c_int32, C.POINTER(_P)]),
    "enn_b200_oplist_last_output_ptr": (C.c_int32, [_P, C.c_int32, C.POINTER(_P)]),
    "enn_b200_oplist_node_count": (C.c_int32, [_P, C.POINTER(C.c_int32)]),
    "enn_b200_oplist_node_info": (C.c_int32, [_P, C.c_int32, C.POINTER(OpInfo), C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    "enn_b200_oplist_profile": (C.c_int32, [_P, C.c_int32, C.POINTER(C.c_float), C.c_int32]),
    "enn_b200_timer_create": (C.c_int32, [_P, C.POINTER(_P)]),
    "enn_b200_timer_start": (C.c_int32, [_P]),
    "enn_b200_timer_stop": (C.c_int32, [_P]),
    "enn_b200_timer_elapsed_us": (C.c_int32, [_P, C.POINTER(C.c_float)]),
    "enn_b200_timer_destroy": (C.c_int32, [_P]),
    "enn_b200_oplist_stats": (C.c_int32, [_P, C.POINTER(C.c_int64), C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    "enn_b200_oplist_destroy": (C.c_int32, [_P]),
    "enn_b200_group_create": (C.c_int32, [C.POINTER(_P), C.c_int32, C.POINTER(_P)]),
    "enn_b200_group_execute": (C.c_int32, [_P, C.POINTER(_P), C.POINTER(_P)]),
    "enn_b200_group_submit": (C.c_int32, [_P, C.POINTER(_P), C.POINTER(_P)]),
    "enn_b200_group_wait": (C.c_int32, [_P]),
    "enn_b200_group_last_error": (C.c_int32, [_P, C.c_char_p, C.c_size_t]),
    "enn_b200_group_destroy": (C.c_int32, [_P, C.c_int32]),
    "enn_b200_model_open": (C.c_int32, [_P, _P, C.c_size_t, C.c_int32, C.POINTER(_P)]),
    "enn_b200_model_info": (C.c_int32, [_P, C.POINTER(C.c_int32), C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    "enn_b200_model_io_bytes": (C.c_int32, [_P, C.c_int32, C.c_int32, C.POINTER(C.c_int64)]),
    "enn_b200_model_oplist": (C.c_int32, [_P, C.POINTER(_P)]),
    "enn_b200_model_execute": (C.c_int32, [_P, C.POINTER(_P), C.POINTER(_P)]),
    "enn_b200_model_close": (C.c_int32, [_P]),
    "enn_b200_nchw_to_nhwc": (C.c_int32, [_P, _P, _P, C.c_int32, C.c_int32, C.c_int32, C.c_int32]),
    "enn_b200_nhwc_to_nchw": (C.c_int32, [_P, _P, _P, C.c_int32, C.c_int32, C.c_int32, C.c_int32]),
    "enn_b200_quantize_multiplier": (None, [C.c_double, C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    "enn_b200_conv_multiplier": (C.c_int32, [C.c_double, C.c_double, C.c_double, C.c_double, C.POINTER(C.c_double)]),
    "enn_b200_activation_range": (None, [C.c_int32, C.c_int32, C.c_float, C.c_int32, C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    "enn_b200_requant_host": (C.c_int32, [C.c_int32] * 6),
    "enn_b200_measure_mma_peak": (C.c_int32, [_P, C.c_int32, C.c_int32, C.c_int32, C.POINTER(C.c_double)]),
    "enn_b200_version": (C.c_char_p, []),
}


def build(verbose=False):
    """Compile libenn_b200.so for sm_100a in-tree (nvcc; works without a GPU)."""
    r = subprocess.run(["make", "-C", _HERE, "-j8"], capture_output=True, text=True)
    if verbose or r.returncode:
        print(r.stdout[-4000:], r.stderr[-4000:])
    if r.returncode:
        raise RuntimeError("building libenn_b200.so failed")


def load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: run `make -C {_HERE}` (there is no CPU fallback)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


lib = load()


class EnnError(RuntimeError):
    def __init__(self, status, msg):
        super().__init__(f"status {status}: {msg}")
        self.status = status


def _np_ptr(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


class Context:
    """One device + one in-order stream (the reference's CLRuntime command queue)."""

    def __init__(self, device=0):
        h = C.c_void_p()
        st = lib.enn_b200_context_create(device, C.byref(h))
        if st != SUCCESS:
            raise EnnError(st, "enn_b200_context_create failed (no CUDA device?)")
        self.h = h
        self.device = device

    def check(self, st):
        if st != SUCCESS:
            buf = C.create_string_buffer(512)
            lib.enn_b200_last_error(self.h, buf, 512)
            raise EnnError(st, buf.value.decode())

    def malloc(self, nbytes):
        p = C.c_void_p()
        self.check(lib.enn_b200_malloc(self.h, nbytes, C.byref(p)))
        return p

    def free(self, p):
        self.check(lib.enn_b200_free(self.h, p))

    def upload(self, dev, arr):
        arr = np.ascontiguousarray(arr)
        self.check(lib.enn_b200_upload(self.h, dev, _np_ptr(arr), arr.nbytes))
        self.sync()  # arr may be a temporary

    def to_device(self, arr):
        arr = np.ascontiguousarray(arr)
        p = self.malloc(arr.nbytes)
        self.upload(p, arr)
        return p

    def download(self, dev, shape, dtype=np.uint8):
        out = np.empty(shape, dtype=dtype)
        self.check(lib.enn_b200_download(self.h, _np_ptr(out), dev, out.nbytes))
        return out

    def sync(self):
        self.check(lib.enn_b200_stream_sync(self.h))

    @property
    def stream(self):
        return lib.enn_b200_stream(self.h)

    def set_option(self, name, value):
        """Planner override for operators prepared afterwards (tests and tuning)."""
        self.check(lib.enn_b200_context_set_option(self.h, name.encode(), int(value)))

    def mma_peak(self, kind=0, n=256, iters=4096):
        """Measured tcgen05.mma rate in tera-ops/s (kind 0: int8, kind 1: bf16)."""
        v = C.c_double()
        self.check(lib.enn_b200_measure_mma_peak(self.h, kind, n, iters, C.byref(v)))
        return v.value

    def close(self):
        if self.h:
            lib.enn_b200_context_destroy(self.h)
            self.h = None


class Op:
    """A prepared operator handle (CLConvolution / CLDepthwiseConvolution / ... after initialize())."""

    def __init__(self, ctx, handle):
        self.ctx, self.h = ctx, handle
        self.info = OpInfo()
        ctx.check(lib.enn_b200_op_info(handle, C.byref(self.info)))

    def set_impl(self, impl):
        self.ctx.check(lib.enn_b200_op_set_impl(self.h, impl))
        self.ctx.check(lib.enn_b200_op_info(self.h, C.byref(self.info)))

    def execute(self, in_dev, out_dev):
        self.ctx.check(lib.enn_b200_op_execute(self.h, in_dev, out_dev))

    def execute2(self, a_dev, b_dev, out_dev):
        self.ctx.check(lib.enn_b200_op_execute2(self.h, a_dev, b_dev, out_dev))

    def rebind_constants(self, weights_dev=None, bias_dev=None):
        """Operators prepared with weights_as_input / bias_as_input: take the tensors' current device contents."""
        self.ctx.check(lib.enn_b200_op_rebind_constants(self.h, weights_dev, bias_dev))

    def fuse_add(self, add_op, conv_is_second_input=False):
        """Moves a prepared add over this convolution's output into its epilogue; the add is owned by this op afterwards.
        Raises EnnError(INVALID_PARAMS) and leaves both untouched when the plan cannot take it."""
        self.ctx.check(lib.enn_b200_op_fuse_add(self.h, add_op.h, int(conv_is_second_input)))
        add_op.h = None
        self.ctx.check(lib.enn_b200_op_info(self.h, C.byref(self.info)))

    def execute_n(self, in_devs, out_dev):
        arr = (C.c_void_p * len(in_devs))(*[p.value if hasattr(p, "value") else p for p in in_devs])
        self.ctx.check(lib.enn_b200_op_execute_n(self.h, arr, len(in_devs), out_dev))

    def run_n(self, xs):
        """Upload several host arrays, execute the n-input form, download."""
        devs = [self.ctx.to_device(x) for x in xs]
        o = self.ctx.malloc(max(1, self.info.out_bytes))
        try:
            self.execute_n(devs, o)
            return self.ctx.download(o, (self.info.out_bytes,), np.int8 if xs[0].dtype == np.int8 else np.uint8)
        finally:
            for p in devs + [o]:
                self.ctx.free(p)

    def test_starve_next(self):
        self.ctx.check(lib.enn_b200_op_test_starve_next(self.h))

    def clear_error(self):
        self.ctx.check(lib.enn_b200_op_clear_error(self.h))

    @property
    def out_shape(self):
        i = self.info
        return (i.out_n, i.out_h, i.out_w, i.out_c)

    def run(self, x, x2=None):
        """Upload host array(s), execute, download: convenience for tests."""
        act = np.int8 if x.dtype == np.int8 else np.uint8
        a = self.ctx.to_device(x)
        b = self.ctx.to_device(x2) if x2 is not None else None
        nbytes = max(1, self.info.out_bytes)
        o = self.ctx.malloc(nbytes)
        try:
            if x2 is None:
                self.execute(a, o)
            else:
                self.execute2(a, b, o)
            return self.ctx.download(o, (self.info.out_bytes,), act)
        finally:
            self.ctx.free(a)
            self.ctx.free(o)
            if b is not None:
                self.ctx.free(b)

    def release(self):
        if self.h:
            lib.enn_b200_op_release(self.h)
            self.h = None


def _prepare(ctx, fn, desc, w, bias, scales):
    h = C.c_void_p()
    w = np.ascontiguousarray(w) if w is not None else None                      # None: weights_as_input
    bias = np.ascontiguousarray(bias, dtype=np.int32) if bias is not None else None  # None: bias_as_input
    sc = np.ascontiguousarray(scales, dtype=np.float32) if scales is not None else None
    ctx.check(fn(ctx.h, C.byref(desc), _np_ptr(w), _np_ptr(bias), _np_ptr(sc), C.byref(h)))
    return Op(ctx, h)


def conv2d(ctx, desc, w, bias, scales=None):
    return _prepare(ctx, lib.enn_b200_conv2d_prepare, desc, w, bias, scales)


def depthwise(ctx, desc, w, bias, scales=None):
    return _prepare(ctx, lib.enn_b200_depthwise_prepare, desc, w, bias, scales)


def deconv(ctx, desc, w, bias, scales=None):
    return _prepare(ctx, lib.enn_b200_deconv_prepare, desc, w, bias, scales)


def fully_connected(ctx, desc, w, bias, scales=None):
    return _prepare(ctx, lib.enn_b200_fc_prepare, desc, w, bias, scales)


def add(ctx, desc):
    h = C.c_void_p()
    ctx.check(lib.enn_b200_add_prepare(ctx.h, C.byref(desc), C.byref(h)))
    return Op(ctx, h)


def avgpool(ctx, desc):
    h = C.c_void_p()
    ctx.check(lib.enn_b200_avgpool_prepare(ctx.h, C.byref(desc), C.byref(h)))
    return Op(ctx, h)


def _prepare_simple(ctx, fn, desc):
    h = C.c_void_p()
    ctx.check(fn(ctx.h, C.byref(desc), C.byref(h)))
    return Op(ctx, h)


def maxpool(ctx, desc):
    return _prepare_simple(ctx, lib.enn_b200_maxpool_prepare, desc)


def mean(ctx, desc):
    return _prepare_simple(ctx, lib.enn_b200_mean_prepare, desc)


def concat(ctx, desc):
    return _prepare_simple(ctx, lib.enn_b200_concat_prepare, desc)


def softmax(ctx, desc):
    return _prepare_simple(ctx, lib.enn_b200_softmax_prepare, desc)


def resize_bilinear(ctx, desc):
    return _prepare_simple(ctx, lib.enn_b200_resize_bilinear_prepare, desc)


class OpList:
    """Operator list with BufferTable-style tensor ids (GpuUserDriver Open/Execute/CloseSubGraph)."""

    def __init__(self, ctx):
        self.ctx = ctx
        h = C.c_void_p()
        ctx.check(lib.enn_b200_oplist_create(ctx.h, C.byref(h)))
        self.h = h
        self.n_in = self.n_out = 0
        self.out_bytes = []

    def tensor(self, nbytes):
        tid = C.c_int32()
        self.ctx.check(lib.enn_b200_oplist_add_tensor(self.h, int(nbytes), C.byref(tid)))
        return tid.value

    def add(self, op, in_ids, out_id):
        ids = (C.c_int32 * len(in_ids))(*in_ids)
        self.ctx.check(lib.enn_b200_oplist_add_op(self.h, op.h, ids, len(in_ids), out_id))
        op.h = None        # owned by the list now

    def set_io(self, inputs, outputs, out_bytes):
        a = (C.c_int32 * len(inputs))(*inputs)
        b = (C.c_int32 * len(outputs))(*outputs)
        self.ctx.check(lib.enn_b200_oplist_set_io(self.h, a, len(inputs), b, len(outputs)))
        self.n_in, self.n_out, self.out_bytes = len(inputs), len(outputs), list(out_bytes)

    def finalize(self):
        self.ctx.check(lib.enn_b200_oplist_finalize(self.h))

    def execute_host_ptrs(self, in_ptrs, out_ptrs):
        a = (C.c_void_p * len(in_ptrs))(*in_ptrs)
        b = (C.c_void_p * len(out_ptrs))(*out_ptrs)
        self.ctx.check(lib.enn_b200_oplist_execute(self.h, a, b))

    def submit_host_ptrs(self, in_ptrs, out_ptrs):
        a = (C.c_void_p * len(in_ptrs))(*in_ptrs)
        b = (C.c_void_p * len(out_ptrs))(*out_ptrs)
        self.ctx.check(lib.enn_b200_oplist_submit(self.h, a, b))

    @staticmethod
    def submit_round(lists, in_ptrs, out_ptrs):
        """One pipelined submission on every list of `lists` (same device), started together; in_ptrs[k] / out_ptrs[k]
        are the host pointer lists of lists[k]."""
        n = len(lists)
        hs = (C.c_void_p * n)(*[l.h for l in lists])
        ins = [(C.c_void_p * len(p))(*p) for p in in_ptrs]
        outs = [(C.c_void_p * len(p))(*p) for p in out_ptrs]
        pin = (C.POINTER(C.c_void_p) * n)(*[C.cast(a, C.POINTER(C.c_void_p)) for a in ins])
        pout = (C.POINTER(C.c_void_p) * n)(*[C.cast(a, C.POINTER(C.c_void_p)) for a in outs])
        lists[0].ctx.check(lib.enn_b200_oplist_submit_round(hs, n, pin, pout))

    def wait(self):
        self.ctx.check(lib.enn_b200_oplist_wait(self.h))

    def execute(self, inputs):
        """inputs: list of numpy arrays; returns list of uint8 arrays (flat)."""
        ins = [np.ascontiguousarray(x) for x in inputs]
        outs = [np.empty(n, np.uint8) for n in self.out_bytes]
        self.execute_host_ptrs([x.ctypes.data for x in ins], [o.ctypes.data for o in outs])
        return outs

    def execute_device(self):
        self.ctx.check(lib.enn_b200_oplist_execute_device(self.h))

    def tensor_ptr(self, tid):
        p = C.c_void_p()
        self.ctx.check(lib.enn_b200_oplist_tensor_ptr(self.h, tid, C.byref(p)))
        return p

    def last_output_ptr(self, index=0):
        p = C.c_void_p()
        self.ctx.check(lib.enn_b200_oplist_last_output_ptr(self.h, index, C.byref(p)))
        return p

    def nodes(self):
        """The nodes after finalize: list of (OpInfo, kind, number of inputs)."""
        n = C.c_int32()
        self.ctx.check(lib.enn_b200_oplist_node_count(self.h, C.byref(n)))
        out = []
        for i in range(n.value):
            info, kind, nin = OpInfo(), C.c_int32(), C.c_int32()
            self.ctx.check(lib.enn_b200_oplist_node_info(self.h, i, C.byref(info), C.byref(kind), C.byref(nin)))
            out.append((info, kind.value, nin.value))
        return out

    def profile(self, repeats=5):
        """Device microseconds per node (eager passes with an event between the nodes)."""
        n = C.c_int32()
        self.ctx.check(lib.enn_b200_oplist_node_count(self.h, C.byref(n)))
        us = (C.c_float * max(1, n.value))()
        self.ctx.check(lib.enn_b200_oplist_profile(self.h, repeats, us, n.value))
        return [us[i] for i in range(n.value)]

    def stats(self):
        a, b, c = C.c_int64(), C.c_int32(), C.c_int32()
        self.ctx.check(lib.enn_b200_oplist_stats(self.h, C.byref(a), C.byref(b), C.byref(c)))
        return {"device_bytes": a.value, "buffers": b.value, "kernel_launches": c.value}

    def destroy(self):
        if self.h:
            lib.enn_b200_oplist_destroy(self.h)
            self.h = None


class Group:
    """One ExecuteSubGraph call over several operator lists (one per device, or several per device): the batch is split
    along its outermost dimension in member order, members run side by side, results land in one host buffer."""

    def __init__(self, lists):
        self.lists = list(lists)
        arr = (C.c_void_p * len(self.lists))(*[l.h for l in self.lists])
        h = C.c_void_p()
        st = lib.enn_b200_group_create(arr, len(self.lists), C.byref(h))
        if st != SUCCESS:
            raise EnnError(st, "enn_b200_group_create failed")
        self.h = h
        self.out_bytes = [sum(l.out_bytes[i] for l in self.lists) for i in range(self.lists[0].n_out)]

    def _check(self, st):
        if st != SUCCESS:
            buf = C.create_string_buffer(512)
            lib.enn_b200_group_last_error(self.h, buf, 512)
            raise EnnError(st, buf.value.decode())

    def execute_host_ptrs(self, in_ptrs, out_ptrs):
        self._check(lib.enn_b200_group_execute(self.h, (C.c_void_p * len(in_ptrs))(*in_ptrs), (C.c_void_p * len(out_ptrs))(*out_ptrs)))

    def submit_host_ptrs(self, in_ptrs, out_ptrs):
        self._check(lib.enn_b200_group_submit(self.h, (C.c_void_p * len(in_ptrs))(*in_ptrs), (C.c_void_p * len(out_ptrs))(*out_ptrs)))

    def wait(self):
        self._check(lib.enn_b200_group_wait(self.h))

    def execute(self, inputs):
        ins = [np.ascontiguousarray(x) for x in inputs]
        outs = [np.empty(n, np.uint8) for n in self.out_bytes]
        self.execute_host_ptrs([x.ctypes.data for x in ins], [o.ctypes.data for o in outs])
        return outs

    def destroy(self, destroy_lists=True):
        if self.h:
            lib.enn_b200_group_destroy(self.h, 1 if destroy_lists else 0)
            self.h = None
            if destroy_lists:
                for l in self.lists:
                    l.h = None


class Model:
    """An NNC (v2) model file opened through the front end: parsed, operators prepared, operator list finalized."""

    def __init__(self, ctx, nnc_bytes, batch=0):
        self.ctx = ctx
        h = C.c_void_p()
        buf = (C.c_uint8 * len(nnc_bytes)).from_buffer_copy(nnc_bytes)
        ctx.check(lib.enn_b200_model_open(ctx.h, buf, len(nnc_bytes), batch, C.byref(h)))
        self.h = h
        a, b, c = C.c_int32(), C.c_int32(), C.c_int32()
        lib.enn_b200_model_info(h, C.byref(a), C.byref(b), C.byref(c))
        self.n_inputs, self.n_outputs, self.n_operators = a.value, b.value, c.value

    def io_bytes(self, is_output, index):
        v = C.c_int64()
        self.ctx.check(lib.enn_b200_model_io_bytes(self.h, int(is_output), index, C.byref(v)))
        return v.value

    def execute(self, inputs):
        ins = [np.ascontiguousarray(x) for x in inputs]
        outs = [np.empty(self.io_bytes(True, i), np.uint8) for i in range(self.n_outputs)]
        a = (C.c_void_p * len(ins))(*[x.ctypes.data for x in ins])
        b = (C.c_void_p * len(outs))(*[o.ctypes.data for o in outs])
        self.ctx.check(lib.enn_b200_model_execute(self.h, a, b))
        return outs

    def close(self):
        if self.h:
            lib.enn_b200_model_close(self.h)
            self.h = None
