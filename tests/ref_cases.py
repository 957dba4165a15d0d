"""Seeded cases shared by the generator of tests/golden/ref_kernels.npz and the tests that replay them."""
import numpy as np

import cases

enn = cases.enn


def _pool(seed, n, h, w, c, k, s, act=0):
    x = np.random.default_rng(seed).integers(0, 256, (n, h, w, c), dtype=np.int64).astype(np.uint8)
    d = enn.PoolDesc(n=n, h=h, w=w, c=c, kh=k, kw=k, stride_h=s, stride_w=s, pad_t=0, pad_l=0, out_h=(h - k) // s + 1,
                     out_w=(w - k) // s + 1, activation=act, act_dtype=enn.U8, out_scale=0.05, out_zp=10)
    return d, x


def _add(seed, count, act=0):
    rng = np.random.default_rng(seed)
    a = rng.integers(0, 256, count, dtype=np.int64).astype(np.uint8)
    b = rng.integers(0, 256, count, dtype=np.int64).astype(np.uint8)
    d = enn.AddDesc(count=count, activation=act, act_dtype=enn.U8, in0_scale=0.031, in0_zp=120, in1_scale=0.047, in1_zp=131,
                    out_scale=0.06, out_zp=126)
    return d, a, b


def _maxpool(seed, n, h, w, c, k, s, pad, act=0):
    x = np.random.default_rng(seed).integers(0, 256, (n, h, w, c), dtype=np.int64).astype(np.uint8)
    oh, ow = (h - k + s + 2 * pad) // s, (w - k + s + 2 * pad) // s          # CLMaxpool.cpp:62-67
    d = enn.PoolDesc(n=n, h=h, w=w, c=c, kh=k, kw=k, stride_h=s, stride_w=s, pad_t=pad, pad_l=pad, out_h=oh, out_w=ow, activation=act,
                     act_dtype=enn.U8, out_scale=0.05, out_zp=10)
    return d, x


def _mean(seed, dims, axes):
    x = np.random.default_rng(seed).integers(0, 256, dims, dtype=np.int64).astype(np.uint8)
    return enn.mean_desc(dims, axes), x


def _concat(seed, outer, inner, scales, zps, out_scale, out_zp):
    rng = np.random.default_rng(seed)
    xs = [rng.integers(0, 256, (outer, k), dtype=np.int64).astype(np.uint8) for k in inner]
    return enn.concat_desc(outer, inner, scales, zps, out_scale, out_zp), xs


def _resize(seed, n, h, w, c, oh, ow, align=0, half=0):
    x = np.random.default_rng(seed).integers(0, 256, (n, h, w, c), dtype=np.int64).astype(np.uint8)
    return enn.ResizeDesc(n=n, h=h, w=w, c=c, out_h=oh, out_w=ow, align_corners=align, half_pixel_centers=half, act_dtype=enn.U8), x


CASES = {
    "conv_pc_3x3": ("conv_pc", lambda: cases.conv_case(seed=101, n=2, h=9, w=10, cin=8, cout=12, k=3, per_channel=True, out_scale=0.2)),
    "conv_pc_1x1_relu6": ("conv_pc", lambda: cases.conv_case(seed=102, n=1, h=7, w=7, cin=32, cout=16, k=1, per_channel=True, out_scale=0.1, out_zp=0)),
    "conv_pc_s2_group": ("conv_pc", lambda: cases.conv_case(seed=103, n=1, h=11, w=9, cin=8, cout=8, k=3, stride=2, groups=2, per_channel=True,
                                                               out_scale=0.15, layout=enn.W_OIHW, act=enn.ACT_NONE)),
    # per-tensor u8 convolution through the reference's GEMM path (pad_opt, convert_optimized / convertBlocked2,
    # alignQuantizedWeight_gemm, quantizedGemmBlocked): the configuration-1 geometry at reduced size, groups, stride 2 with
    # a reduction length that is not a multiple of 16, 1x1 with a small weight zero point, a 7x7 first layer
    "conv_pt_config1_14": ("conv_pt", lambda: cases.conv_case(seed=120, n=1, h=14, w=14, cin=64, cout=64, k=3)),
    "conv_pt_groups": ("conv_pt", lambda: cases.conv_case(seed=121, n=2, h=9, w=9, cin=8, cout=12, k=3, groups=4, layout=enn.W_OIHW)),
    "conv_pt_s2_ragged": ("conv_pt", lambda: cases.conv_case(seed=122, n=2, h=9, w=11, cin=5, cout=7, k=3, stride=2, w_zp=140, act=enn.ACT_RELU)),
    "conv_pt_1x1_zp3": ("conv_pt", lambda: cases.conv_case(seed=123, n=1, h=7, w=7, cin=24, cout=10, k=1, w_zp=3, act=enn.ACT_NONE)),
    "conv_pt_7x7_s2": ("conv_pt", lambda: cases.conv_case(seed=124, n=1, h=33, w=35, cin=3, cout=5, k=7, stride=2, w_zp=200)),
    "dw_pc_s1": ("dw", lambda: cases.depthwise_case(seed=104, n=2, h=12, w=12, c=8)),
    "dw_pc_s2": ("dw", lambda: cases.depthwise_case(seed=105, n=1, h=13, w=11, c=12, stride=2)),
    "dw_pt_s1": ("dw", lambda: cases.depthwise_case(seed=106, n=1, h=10, w=10, c=8, per_channel=False, out_scale=0.08, out_zp=3)),
    "dw_pt_dm2_5x5": ("dw", lambda: cases.depthwise_case(seed=107, n=1, h=9, w=9, c=4, dm=2, k=5, per_channel=False, out_scale=0.2, out_zp=7,
                                                           act=enn.ACT_NONE)),
    # output channels past cin * depth_multiplier: bias only (depthwise_conv_unequal; one image, as the kernel indexes)
    "dw_pt_unequal": ("dw", lambda: cases.depthwise_case(seed=131, n=1, h=8, w=9, c=6, dm=2, per_channel=False, out_scale=0.3, out_zp=90,
                                                           act=enn.ACT_NONE, extra_out=5)),
    "deconv_pt_4x4s2": ("deconv", lambda: cases.deconv_case(seed=108, n=2, h=6, w=5, cin=16, cout=8)),
    "deconv_pt_ohwi_relu6": ("deconv", lambda: cases.deconv_case(seed=109, n=1, h=5, w=5, cin=8, cout=4, layout=enn.W_OHWI, act=enn.ACT_RELU6)),
    "deconv_pc_3x3s2": ("deconv", lambda: cases.deconv_case(seed=110, n=1, h=5, w=6, cin=12, cout=8, k=3, stride=2, pad=0, per_channel=True,
                                                              out_scale=0.5)),
    "avgpool_7x7": ("pool", lambda: _pool(111, 2, 7, 7, 16, 7, 1)),
    "avgpool_3x3s2": ("pool", lambda: _pool(112, 1, 9, 9, 8, 3, 2, act=enn.ACT_RELU6)),
    "add": ("add", lambda: _add(113, 4099)),
    "add_relu6": ("add", lambda: _add(114, 1000, act=enn.ACT_RELU6)),
    # remaining graph operators: maxpooling, mean (global-pool form and the halving sum_axis form), concat_axis1 with equal and
    # different scales, resize_bilinear in its three coordinate conventions
    "maxpool_3x3s2_pad": ("maxpool", lambda: _maxpool(130, 2, 9, 11, 6, 3, 2, 1)),
    "maxpool_2x2_relu6": ("maxpool", lambda: _maxpool(131, 1, 8, 8, 16, 2, 2, 0, act=enn.ACT_RELU6)),
    "mean_hw_nhwc": ("mean", lambda: _mean(132, (2, 7, 7, 12), (1, 2))),
    "mean_trailing": ("mean", lambda: _mean(133, (3, 5, 6, 9), (2, 3))),
    "mean_single_axis": ("mean", lambda: _mean(134, (2, 4, 10, 3), (2,))),
    "concat_mixed_scales": ("concat", lambda: _concat(135, 30, (5, 8, 3), (0.02, 0.031, 0.02), (3, 120, 7), 0.02, 11)),
    "resize_up": ("resize", lambda: _resize(136, 2, 5, 6, 4, 10, 13)),
    "resize_align_corners": ("resize", lambda: _resize(137, 1, 7, 7, 3, 13, 9, align=1)),
    "resize_half_pixel_down": ("resize", lambda: _resize(138, 1, 9, 8, 2, 4, 5, half=1)),
}


def run_reference(orc, kind, case):
    if kind == "conv_pc":
        d, x, w, b, sc = case
        return orc.ref_conv_per_channel(d, x, w, b, sc)
    if kind == "conv_pt":
        d, x, w, b, sc = case
        return orc.ref_conv_per_tensor(d, x, w, b)
    if kind == "dw":
        d, x, w, b, sc = case
        return orc.ref_depthwise(d, x, w, b, sc)
    if kind == "deconv":
        d, x, w, b, sc = case
        return orc.ref_deconv(d, x, w, b, sc)
    if kind == "pool":
        d, x = case
        return orc.ref_avgpool(d, x)
    if kind == "maxpool":
        return orc.ref_maxpool(*case)
    if kind == "mean":
        return orc.ref_mean(*case)
    if kind == "resize":
        return orc.ref_resize_bilinear(*case)
    if kind == "concat":
        # the reference concatenates NCHW tensors along C: present the [outer][inner_i] inputs as [1][inner_i][outer]
        d, xs = case
        n = d.n_inputs
        out = orc.ref_concat_channels_nchw([np.ascontiguousarray(x.T[None]) for x in xs], [d.in_scale[i] for i in range(n)],
                                           [d.in_zp[i] for i in range(n)], d.out_scale, d.out_zp)
        return np.ascontiguousarray(out[0].T)
    d, a, b = case
    return orc.ref_add(d, a, b)


def run_oracle(orc, kind, case):
    if kind in ("conv_pc", "conv_pt"):
        d, x, w, b, sc = case
        return orc.conv2d(d, x, w, b, sc)
    if kind == "dw":
        d, x, w, b, sc = case
        return orc.depthwise(d, x, w, b, sc)
    if kind == "deconv":
        d, x, w, b, sc = case
        return orc.deconv(d, x, w, b, sc)
    if kind == "pool":
        d, x = case
        return orc.avgpool(d, x)
    if kind == "maxpool":
        return orc.maxpool(*case)
    if kind == "mean":
        return orc.mean(*case)
    if kind == "resize":
        return orc.resize_bilinear(*case)
    if kind == "concat":
        return orc.concat(*case)
    d, a, b = case
    return orc.add(d, a, b)
