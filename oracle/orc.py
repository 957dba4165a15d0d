"""ctypes wrapper of the CPU oracle (oracle/liboracle.so) and, when built, of the reference's own host
code (oracle/_ref/libennref.so).  TEST INFRASTRUCTURE ONLY: imported by tests/, the smoke test and the
benchmark's CPU-baseline leg, never by the library."""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "liboracle.so")
_REF = os.path.join(_HERE, "_ref", "libennref.so")


def build():
    r = subprocess.run(["make", "-C", _HERE], capture_output=True, text=True)
    if r.returncode:
        raise RuntimeError("building the oracle failed:\n" + r.stdout[-3000:] + r.stderr[-3000:])


if not os.path.exists(_LIB):
    build()
lib = C.CDLL(_LIB)
ref = C.CDLL(_REF) if os.path.exists(_REF) else None

_i32, _p, _f, _d = C.c_int32, C.c_void_p, C.c_float, C.c_double
_pi32 = C.POINTER(C.c_int32)
for _l, _pre in ((lib, "orc_"), (ref, "ref_")):
    if _l is None:
        continue
    getattr(_l, _pre + "quantize_multiplier").argtypes = [_d, _pi32, _pi32]
    getattr(_l, _pre + "quantize_multiplier").restype = None
    getattr(_l, _pre + "conv_multiplier").argtypes = [_d, _d, _d, _d, C.POINTER(_d)]
    getattr(_l, _pre + "conv_multiplier").restype = _i32
    getattr(_l, _pre + "activation_range").argtypes = [_i32, _i32, _f, _i32, _pi32, _pi32]
    getattr(_l, _pre + "activation_range").restype = None
    getattr(_l, _pre + "srdhm").argtypes = [_i32, _i32]
    getattr(_l, _pre + "srdhm").restype = _i32
    getattr(_l, _pre + "rdivpot").argtypes = [_i32, _i32]
    getattr(_l, _pre + "rdivpot").restype = _i32
lib.orc_requant.argtypes = [_i32] * 6
lib.orc_requant.restype = _i32
lib.orc_num_threads.restype = _i32
if ref is not None:
    ref.ref_multiply_by_quantized_multiplier.argtypes = [_i32, _i32, _i32]
    ref.ref_multiply_by_quantized_multiplier.restype = _i32


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def quantize_multiplier(m, which=None):
    l, pre = (which or lib), ("orc_" if (which or lib) is lib else "ref_")
    qm, sh = C.c_int32(), C.c_int32()
    getattr(l, pre + "quantize_multiplier")(m, C.byref(qm), C.byref(sh))
    return qm.value, sh.value


def conv_multiplier(a, b, c, d, which=None):
    l, pre = (which or lib), ("orc_" if (which or lib) is lib else "ref_")
    m = C.c_double(0.0)
    st = getattr(l, pre + "conv_multiplier")(a, b, c, d, C.byref(m))
    return st, m.value


def activation_range(act, dtype, scale, zp, which=None):
    l, pre = (which or lib), ("orc_" if (which or lib) is lib else "ref_")
    lo, hi = C.c_int32(), C.c_int32()
    getattr(l, pre + "activation_range")(act, dtype, scale, zp, C.byref(lo), C.byref(hi))
    return lo.value, hi.value


def _act_np(dtype):
    return np.int8 if dtype == 1 else np.uint8


def _run_conv_like(fn, dims_fn, desc, x, w, bias, scales):
    oh, ow = C.c_int32(), C.c_int32()
    dims_fn(C.byref(desc), C.byref(oh), C.byref(ow))
    x = np.ascontiguousarray(x)
    w = np.ascontiguousarray(w)
    bias = np.ascontiguousarray(bias, dtype=np.int32)
    sc = np.ascontiguousarray(scales, dtype=np.float32) if scales is not None else None
    out = np.empty((desc.n, oh.value, ow.value, desc.cout), dtype=_act_np(desc.act_dtype))
    st = fn(C.byref(desc), _ptr(x), _ptr(w), _ptr(bias), _ptr(sc), _ptr(out))
    assert st == 0
    return out


def conv2d(desc, x, w, bias, scales=None):
    return _run_conv_like(lib.orc_conv2d, lib.orc_conv_out_dims, desc, x, w, bias, scales)


def depthwise(desc, x, w, bias, scales=None):
    return _run_conv_like(lib.orc_depthwise, lib.orc_conv_out_dims, desc, x, w, bias, scales)


def deconv(desc, x, w, bias, scales=None):
    return _run_conv_like(lib.orc_deconv, lib.orc_deconv_out_dims, desc, x, w, bias, scales)


def fully_connected(desc, x, w, bias, scales=None, float_emulation=False):
    x = np.ascontiguousarray(x)
    w = np.ascontiguousarray(w)
    bias = np.ascontiguousarray(bias, dtype=np.int32)
    sc = np.ascontiguousarray(scales, dtype=np.float32) if scales is not None else None
    out = np.empty((desc.m, desc.n), dtype=_act_np(desc.act_dtype))
    if float_emulation:
        st = lib.orc_fc_float(C.byref(desc), _ptr(x), _ptr(w), _ptr(bias), _ptr(out))
    else:
        st = lib.orc_fc(C.byref(desc), _ptr(x), _ptr(w), _ptr(bias), _ptr(sc), _ptr(out))
    assert st == 0
    return out


def add(desc, a, b):
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    out = np.empty(a.shape, dtype=a.dtype)
    st = lib.orc_add(C.byref(desc), _ptr(a), _ptr(b), _ptr(out))
    if st:
        raise ValueError(f"orc_add rejected the parameters ({st})")
    return out


def avgpool(desc, x):
    x = np.ascontiguousarray(x)
    out = np.empty((desc.n, desc.out_h, desc.out_w, desc.c), dtype=x.dtype)
    st = lib.orc_avgpool(C.byref(desc), _ptr(x), _ptr(out))
    assert st == 0
    return out


def maxpool(desc, x):
    x = np.ascontiguousarray(x)
    out = np.empty((desc.n, desc.out_h, desc.out_w, desc.c), dtype=x.dtype)
    assert lib.orc_maxpool(C.byref(desc), _ptr(x), _ptr(out)) == 0
    return out


def mean(desc, x):
    x = np.ascontiguousarray(x)
    shape = [1 if desc.axis_mask & (1 << a) else desc.dims[a] for a in range(4)]
    out = np.empty(shape, dtype=x.dtype)
    assert lib.orc_mean(C.byref(desc), _ptr(x), _ptr(out)) == 0
    return out


def concat(desc, xs):
    xs = [np.ascontiguousarray(x) for x in xs]
    total = sum(desc.inner[i] for i in range(desc.n_inputs))
    out = np.empty((desc.outer, total), dtype=xs[0].dtype)
    arr = (C.c_void_p * len(xs))(*[x.ctypes.data for x in xs])
    assert lib.orc_concat(C.byref(desc), arr, _ptr(out)) == 0
    return out


def softmax(desc, x):
    x = np.ascontiguousarray(x)
    out = np.empty(x.shape, dtype=x.dtype)
    assert lib.orc_softmax(C.byref(desc), _ptr(x), _ptr(out)) == 0
    return out


def resize_bilinear(desc, x):
    x = np.ascontiguousarray(x)
    out = np.empty((desc.n, desc.out_h, desc.out_w, desc.c), dtype=x.dtype)
    assert lib.orc_resize_bilinear(C.byref(desc), _ptr(x), _ptr(out)) == 0
    return out


def num_threads():
    return lib.orc_num_threads()


def set_num_threads(n):
    lib.orc_set_num_threads(int(n))


# ---- the reference's own kernel text compiled as C++ (oracle/ref_kernels_shim.cpp), when built ----
def has_ref_kernels():
    return ref is not None and hasattr(ref, "ref_has_kernels")


def _ref_conv_like(fn, dims_fn, desc, x, w, bias, scales):
    oh, ow = C.c_int32(), C.c_int32()
    dims_fn(C.byref(desc), C.byref(oh), C.byref(ow))
    x = np.ascontiguousarray(x)
    w = np.ascontiguousarray(w)
    bias = np.ascontiguousarray(bias, dtype=np.int32)
    sc = np.ascontiguousarray(scales, dtype=np.float32) if scales is not None else None
    out = np.empty((desc.n, oh.value, ow.value, desc.cout), dtype=np.uint8)
    st = fn(C.byref(desc), _ptr(x), _ptr(w), _ptr(bias), _ptr(sc), _ptr(out))
    if st:
        raise ValueError(f"reference kernel wrapper rejected the case ({st})")
    return out


def ref_conv_per_channel(desc, x, w, bias, scales):
    return _ref_conv_like(ref.ref_conv_per_channel, lib.orc_conv_out_dims, desc, x, w, bias, scales)


def ref_conv_per_tensor(desc, x, w, bias):
    """Per-tensor u8 convolution through the reference's own GEMM path (pad_opt, convert_optimized / convertBlocked2,
    alignQuantizedWeight_gemm, quantizedGemmBlocked)."""
    return _ref_conv_like(lambda d, a, b, c, _s, o: ref.ref_conv_per_tensor(d, a, b, c, o), lib.orc_conv_out_dims, desc, x, w, bias, None)


def ref_depthwise(desc, x, w, bias, scales=None):
    return _ref_conv_like(ref.ref_depthwise, lib.orc_conv_out_dims, desc, x, w, bias, scales)


def ref_deconv(desc, x, w, bias, scales=None):
    return _ref_conv_like(ref.ref_deconv, lib.orc_deconv_out_dims, desc, x, w, bias, scales)


def ref_avgpool(desc, x):
    x = np.ascontiguousarray(x)
    out = np.empty((desc.n, desc.out_h, desc.out_w, desc.c), dtype=np.uint8)
    assert ref.ref_avgpool(C.byref(desc), _ptr(x), _ptr(out)) == 0
    return out


def ref_add(desc, a, b):
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    out = np.empty(a.shape, dtype=np.uint8)
    assert ref.ref_add(C.byref(desc), _ptr(a), _ptr(b), _ptr(out)) == 0
    return out


def ref_maxpool(desc, x):
    x = np.ascontiguousarray(x)
    out = np.empty((desc.n, desc.out_h, desc.out_w, desc.c), dtype=np.uint8)
    assert ref.ref_maxpool(C.byref(desc), _ptr(x), _ptr(out)) == 0
    return out


def ref_mean(desc, x):
    """The reference's CLMean on the same dims and axes (its kernels index dims as N, C, H, W; the arithmetic does not
    depend on the names)."""
    x = np.ascontiguousarray(x)
    shape = [1 if desc.axis_mask & (1 << a) else desc.dims[a] for a in range(4)]
    out = np.zeros(shape, dtype=np.uint8)
    assert ref.ref_mean(desc.dims, C.c_int32(desc.axis_mask), _ptr(x), _ptr(out)) == 0
    return out


def ref_concat_channels_nchw(xs, in_scale, in_zp, out_scale, out_zp):
    """Reference concat_axis1 on NCHW inputs [N][C_i][H*W]; returns [N][sum C][H*W]."""
    xs = [np.ascontiguousarray(x) for x in xs]
    n, hw = xs[0].shape[0], xs[0].shape[2]
    ch = (C.c_int32 * len(xs))(*[x.shape[1] for x in xs])
    sc = (C.c_float * len(xs))(*in_scale)
    zp = (C.c_int32 * len(xs))(*in_zp)
    arr = (C.c_void_p * len(xs))(*[x.ctypes.data for x in xs])
    out = np.zeros((n, sum(x.shape[1] for x in xs), hw), np.uint8)
    ref.ref_concat_axis1.argtypes = [C.c_int32, C.c_int32, C.POINTER(C.c_int32), C.c_int32, C.POINTER(C.c_float), C.POINTER(C.c_int32),
                                     C.c_float, C.c_int32, C.POINTER(C.c_void_p), C.c_void_p]
    assert ref.ref_concat_axis1(len(xs), n, ch, hw, sc, zp, out_scale, out_zp, arr, _ptr(out)) == 0
    return out


def ref_resize_bilinear(desc, x):
    x = np.ascontiguousarray(x)
    out = np.empty((desc.n, desc.out_h, desc.out_w, desc.c), dtype=np.uint8)
    assert ref.ref_resize_bilinear(C.byref(desc), _ptr(x), _ptr(out)) == 0
    return out
