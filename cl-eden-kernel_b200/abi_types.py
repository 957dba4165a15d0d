"""Constants and POD descriptors of the C ABI (include/enn_b200.h) as ctypes structures.

Pure declarations: importing this module loads no shared library, so the CPU oracle and the benchmark's CPU arm can
build the same descriptors the CUDA path takes without touching it.
"""
import ctypes as C

import numpy as np

SUCCESS, FAILURE, CUDA_FAILURE, INVALID_PARAMS = 0, 1, 2, 3
ACT_NONE, ACT_RELU, ACT_RELU1, ACT_RELU6 = 0, 1, 2, 3
U8, S8 = 0, 1
W_OIHW, W_OHWI, W_IOHW = 0, 1, 2
IMPL_DIRECT, IMPL_TCGEN05, IMPL_GEMV, IMPL_DEPTHWISE, IMPL_ELTWISE = 0, 1, 2, 3, 4


class ConvDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in (
        "n", "h", "w", "cin", "cout", "kh", "kw", "stride_h", "stride_w", "dil_h", "dil_w",
        "pad_t", "pad_r", "pad_b", "pad_l", "groups", "activation", "act_dtype", "weight_dtype",
        "weight_layout", "per_channel")] + [
        ("in_scale", C.c_float), ("in_zp", C.c_int32), ("w_scale", C.c_float), ("w_zp", C.c_int32),
        ("bias_scale", C.c_float), ("out_scale", C.c_float), ("out_zp", C.c_int32),
        ("out_h", C.c_int32), ("out_w", C.c_int32), ("weights_as_input", C.c_int32), ("bias_as_input", C.c_int32)]


class FcDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("m", "k", "n", "activation", "act_dtype", "weight_dtype", "per_channel")] + [
        ("in_scale", C.c_float), ("in_zp", C.c_int32), ("w_scale", C.c_float), ("w_zp", C.c_int32),
        ("bias_scale", C.c_float), ("out_scale", C.c_float), ("out_zp", C.c_int32),
        ("weights_as_input", C.c_int32), ("bias_as_input", C.c_int32)]


class AddDesc(C.Structure):
    _fields_ = [("count", C.c_int64), ("activation", C.c_int32), ("act_dtype", C.c_int32),
                ("in0_scale", C.c_float), ("in0_zp", C.c_int32), ("in1_scale", C.c_float), ("in1_zp", C.c_int32),
                ("out_scale", C.c_float), ("out_zp", C.c_int32)]


class PoolDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n", "h", "w", "c", "kh", "kw", "stride_h", "stride_w", "pad_t", "pad_l",
                                          "out_h", "out_w", "activation", "act_dtype")] + [
        ("out_scale", C.c_float), ("out_zp", C.c_int32)]


class MeanDesc(C.Structure):
    _fields_ = [("dims", C.c_int32 * 4), ("axis_mask", C.c_int32), ("act_dtype", C.c_int32)]


CONCAT_MAX_INPUTS = 8


class ConcatDesc(C.Structure):
    _fields_ = [("n_inputs", C.c_int32), ("act_dtype", C.c_int32), ("outer", C.c_int64), ("inner", C.c_int64 * CONCAT_MAX_INPUTS),
                ("in_scale", C.c_float * CONCAT_MAX_INPUTS), ("in_zp", C.c_int32 * CONCAT_MAX_INPUTS), ("out_scale", C.c_float),
                ("out_zp", C.c_int32)]


class SoftmaxDesc(C.Structure):
    _fields_ = [("outer", C.c_int64), ("channels", C.c_int32), ("inner", C.c_int64), ("beta", C.c_float), ("act_dtype", C.c_int32),
                ("in_scale", C.c_float), ("in_zp", C.c_int32), ("out_scale", C.c_float), ("out_zp", C.c_int32)]


class ResizeDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n", "h", "w", "c", "out_h", "out_w", "align_corners", "half_pixel_centers", "act_dtype")]


def mean_desc(dims, axes, act_dtype=U8):
    d = MeanDesc()
    for i, v in enumerate(dims):
        d.dims[i] = v
    d.axis_mask = sum(1 << a for a in axes)
    d.act_dtype = act_dtype
    return d


def concat_desc(outer, inner, in_scale, in_zp, out_scale, out_zp, act_dtype=U8):
    d = ConcatDesc()
    d.n_inputs, d.act_dtype, d.outer, d.out_scale, d.out_zp = len(inner), act_dtype, outer, out_scale, out_zp
    for i in range(len(inner)):
        d.inner[i], d.in_scale[i], d.in_zp[i] = inner[i], in_scale[i], in_zp[i]
    return d


class OpInfo(C.Structure):
    _fields_ = [("impl", C.c_int32), ("out_n", C.c_int32), ("out_h", C.c_int32), ("out_w", C.c_int32),
                ("out_c", C.c_int32), ("in_bytes", C.c_int64), ("out_bytes", C.c_int64), ("macs", C.c_int64),
                ("algorithmic_bytes", C.c_int64), ("act_min", C.c_int32), ("act_max", C.c_int32),
                ("kernel_launches", C.c_int32)]


def conv_desc(**kw):
    """ConvDesc with the reference's defaults (stride/dilation 1, one group, no activation, u8/u8, OHWI)."""
    d = ConvDesc()
    d.stride_h = d.stride_w = d.dil_h = d.dil_w = 1
    d.groups = 1
    d.weight_layout = W_OHWI
    d.in_scale = d.w_scale = d.out_scale = 1.0
    d.bias_scale = 1.0
    for k, v in kw.items():
        if not hasattr(d, k):
            raise AttributeError(k)
        setattr(d, k, v)
    if "bias_scale" not in kw:
        d.bias_scale = np.float32(d.in_scale) * np.float32(d.w_scale)
    return d
