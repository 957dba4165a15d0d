"""Seeded synthetic operator workloads: the benchmark configurations and the cases the parity tests draw from.

The reference neither ships nor names a dataset for this path; inputs are drawn with
numpy.random.default_rng(seed) in the order input -> weights -> bias -> scales, with the shapes and value
distributions of the benchmark configurations.  Only descriptors and numpy arrays are produced here: nothing in
this module touches the CUDA library, so the CPU oracle can consume the same cases.
"""
import numpy as np

try:
    from . import abi_types as enn
except ImportError:                   # loaded as a plain module with its directory on sys.path
    import abi_types as enn


def same_pad_tf(in_size, k, s, d=1):
    """TensorFlow-style SAME split used for non-Caffe models (gpu_op_constructor.cc:1997-2004)."""
    out = (in_size + s - 1) // s
    total = max(0, (out - 1) * s + (k - 1) * d + 1 - in_size)
    return total // 2, (total + 1) // 2


def conv_case(seed=0, n=1, h=56, w=56, cin=64, cout=64, k=3, stride=1, dil=1, groups=1, per_channel=False,
              act=enn.ACT_RELU6, layout=enn.W_OHWI, in_scale=0.02, in_zp=128, w_scale=0.005, w_zp=127,
              out_scale=0.05, out_zp=128, pad="same", act_dtype=enn.U8, bias_range=1000, kh=None, kw=None):
    rng = np.random.default_rng(seed)
    kh = kh or k
    kw = kw or k
    cin_g = cin // groups
    if act_dtype == enn.S8:
        x = rng.integers(-128, 128, (n, h, w, cin), dtype=np.int64).astype(np.int8)
    else:
        x = rng.integers(0, 256, (n, h, w, cin), dtype=np.int64).astype(np.uint8)
    wshape = {enn.W_OHWI: (cout, kh, kw, cin_g), enn.W_OIHW: (cout, cin_g, kh, kw)}[layout]
    if per_channel:
        wt = rng.integers(-127, 128, wshape, dtype=np.int64).astype(np.int8)
    else:
        wt = rng.integers(0, 256, wshape, dtype=np.int64).astype(np.uint8)
    bias = rng.integers(-bias_range, bias_range + 1, (cout,), dtype=np.int64).astype(np.int32)
    scales = None
    if per_channel:
        scales = np.exp(rng.uniform(np.log(1e-3), np.log(1e-1), cout)).astype(np.float32)
    if pad == "same":
        pt, pb = same_pad_tf(h, kh, stride, dil)
        pl, pr = same_pad_tf(w, kw, stride, dil)
    elif pad == "valid":
        pt = pb = pl = pr = 0
    else:
        pt, pr, pb, pl = pad
    d = enn.conv_desc(n=n, h=h, w=w, cin=cin, cout=cout, kh=kh, kw=kw, stride_h=stride, stride_w=stride,
                      dil_h=dil, dil_w=dil, pad_t=pt, pad_r=pr, pad_b=pb, pad_l=pl, groups=groups, activation=act,
                      act_dtype=act_dtype, weight_dtype=enn.S8 if per_channel else enn.U8, weight_layout=layout,
                      per_channel=int(per_channel), in_scale=in_scale, in_zp=in_zp, w_scale=w_scale,
                      w_zp=0 if per_channel else w_zp, out_scale=out_scale, out_zp=out_zp)
    return d, x, wt, bias, scales


def depthwise_case(seed=0, n=2, h=112, w=112, c=32, k=3, stride=1, dm=1, per_channel=True, act=enn.ACT_RELU6,
                   layout=enn.W_OIHW, in_scale=0.02, in_zp=128, out_scale=0.04, out_zp=0, dil=1, w_scale=0.01,
                   w_zp=121, act_dtype=enn.U8, extra_out=0):
    """extra_out: output channels past c * dm, which have no filter and carry the requantised bias only
    (depthwise_conv_unequal); bias and per-channel scales cover them, the filter does not."""
    rng = np.random.default_rng(seed)
    cout = c * dm
    if act_dtype == enn.S8:
        x = rng.integers(-128, 128, (n, h, w, c), dtype=np.int64).astype(np.int8)
    else:
        x = rng.integers(0, 256, (n, h, w, c), dtype=np.int64).astype(np.uint8)
    wshape = (cout, 1, k, k) if layout == enn.W_OIHW else (1, k, k, cout)
    if per_channel:
        wt = rng.integers(-127, 128, wshape, dtype=np.int64).astype(np.int8)
    else:
        wt = rng.integers(0, 256, wshape, dtype=np.int64).astype(np.uint8)
    cout += extra_out
    bias = rng.integers(-500 if not extra_out else -40000, 501 if not extra_out else 40001, (cout,), dtype=np.int64).astype(np.int32)
    scales = np.exp(rng.uniform(np.log(1e-3), np.log(1e-1), cout)).astype(np.float32) if per_channel else None
    pt, pb = same_pad_tf(h, k, stride, dil)
    pl, pr = same_pad_tf(w, k, stride, dil)
    d = enn.conv_desc(n=n, h=h, w=w, cin=c, cout=cout, kh=k, kw=k, stride_h=stride, stride_w=stride, dil_h=dil,
                      dil_w=dil, pad_t=pt, pad_r=pr, pad_b=pb, pad_l=pl, groups=dm, activation=act, act_dtype=act_dtype,
                      weight_dtype=enn.S8 if per_channel else enn.U8, weight_layout=layout,
                      per_channel=int(per_channel), in_scale=in_scale, in_zp=in_zp, w_scale=w_scale,
                      w_zp=0 if per_channel else w_zp, out_scale=out_scale, out_zp=out_zp)
    return d, x, wt, bias, scales


def deconv_case(seed=0, n=1, h=16, w=16, cin=128, cout=64, k=4, stride=2, pad=1, per_channel=False,
                layout=enn.W_IOHW, in_scale=0.02, in_zp=128, w_scale=0.004, w_zp=120, out_scale=0.05, out_zp=128,
                act=enn.ACT_NONE, act_dtype=enn.U8):
    rng = np.random.default_rng(seed)
    if act_dtype == enn.S8:
        x = rng.integers(-128, 128, (n, h, w, cin), dtype=np.int64).astype(np.int8)
    else:
        x = rng.integers(0, 256, (n, h, w, cin), dtype=np.int64).astype(np.uint8)
    wshape = (cin, cout, k, k) if layout == enn.W_IOHW else (cout, k, k, cin)
    if per_channel:
        wt = rng.integers(-127, 128, wshape, dtype=np.int64).astype(np.int8)
    else:
        wt = rng.integers(0, 256, wshape, dtype=np.int64).astype(np.uint8)
    bias = rng.integers(-1000, 1001, (cout,), dtype=np.int64).astype(np.int32)
    scales = np.exp(rng.uniform(np.log(1e-3), np.log(1e-1), cout)).astype(np.float32) if per_channel else None
    d = enn.conv_desc(n=n, h=h, w=w, cin=cin, cout=cout, kh=k, kw=k, stride_h=stride, stride_w=stride, pad_t=pad,
                      pad_r=pad, pad_b=pad, pad_l=pad, groups=1, activation=act, act_dtype=act_dtype,
                      weight_dtype=enn.S8 if per_channel else enn.U8, weight_layout=layout,
                      per_channel=int(per_channel), in_scale=in_scale, in_zp=in_zp, w_scale=w_scale,
                      w_zp=0 if per_channel else w_zp, out_scale=out_scale, out_zp=out_zp)
    return d, x, wt, bias, scales


def fc_out_scale(k, in_scale=0.02, w_scale_typ=0.01):
    """Output scale that keeps most outputs unsaturated: ~4 sigma of the accumulator over 127 levels."""
    sigma_acc = np.sqrt(k) * 73.9 * 73.3          # std of U[0,255]-128 times std of U[-127,127]
    return float(np.float32(4.0 * sigma_acc * in_scale * w_scale_typ / 127.0))


def fc_case(seed=0, m=4, k=256, n=64, per_channel=True, act=enn.ACT_NONE, in_scale=0.02, in_zp=128, out_zp=128,
            w_scale=0.01, w_zp=0, out_scale=None, act_dtype=enn.U8):
    rng = np.random.default_rng(seed)
    if act_dtype == enn.S8:
        x = rng.integers(-128, 128, (m, k), dtype=np.int64).astype(np.int8)
    else:
        x = rng.integers(0, 256, (m, k), dtype=np.int64).astype(np.uint8)
    if per_channel:
        wt = rng.integers(-127, 128, (n, k), dtype=np.int64).astype(np.int8)
    else:
        wt = rng.integers(0, 256, (n, k), dtype=np.int64).astype(np.uint8)
        w_zp = w_zp or 127
    bias = rng.integers(-1000, 1001, (n,), dtype=np.int64).astype(np.int32)
    scales = np.exp(rng.uniform(np.log(1e-3), np.log(1e-1), n)).astype(np.float32) if per_channel else None
    d = enn.FcDesc(m=m, k=k, n=n, activation=act, act_dtype=act_dtype, weight_dtype=enn.S8 if per_channel else enn.U8,
                   per_channel=int(per_channel), in_scale=in_scale, in_zp=in_zp, w_scale=w_scale, w_zp=w_zp,
                   bias_scale=float(np.float32(in_scale) * np.float32(w_scale)), out_scale=out_scale or fc_out_scale(k),
                   out_zp=out_zp)
    return d, x, wt, bias, scales
