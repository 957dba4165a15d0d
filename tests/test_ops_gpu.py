"""GPU parity tests: every operator through the C ABI against the CPU oracle, bit for bit."""
import json
import os
import zlib

import numpy as np
import pytest

import cases

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _seed(name):
    """Case seed from the case name, the same in every process (str hashes are randomised per process)."""
    return zlib.crc32(name.encode()) % 1000


def _check(op, y_ref, x, x2=None):
    y = op.run(x, x2).reshape(y_ref.shape)
    bad = np.nonzero(y != y_ref)
    assert bad[0].size == 0, f"{bad[0].size} of {y.size} differ; first at {[int(b[0]) for b in bad]}: " \
                             f"got {y[tuple(b[0] for b in bad)]} want {y_ref[tuple(b[0] for b in bad)]}"


def _impls(enn, op):
    """Every kernel family this op can run with (direct always; tensor core when planned)."""
    out = [op.info.impl]
    for impl in (enn.IMPL_DIRECT, enn.IMPL_TCGEN05):
        if impl not in out:
            try:
                op.set_impl(impl)
                out.append(impl)
            except enn.EnnError:
                pass
    return out


CONV_CASES = {
    "config1_3x3_64": dict(),
    "ragged_5x7": dict(n=2, h=5, w=7, cin=3, cout=5, k=3),
    "stride2": dict(n=2, h=15, w=14, cin=8, cout=12, k=3, stride=2),
    "dilated": dict(n=1, h=13, w=13, cin=8, cout=8, k=3, dil=2),
    "grouped_oihw": dict(n=2, h=9, w=9, cin=8, cout=12, k=3, groups=4, layout=cases.enn.W_OIHW),
    # grouped convolutions on the tensor-core path (block-diagonal weights): gathered 3x3 stride 2, implicit 3x3, in-place 1x1,
    # u8 per-tensor weights (row-sum correction over the zero-point blocks) and int8 per-channel weights
    "grouped_tc_gather_s2": dict(n=2, h=17, w=15, cin=24, cout=36, k=3, stride=2, groups=3, w_zp=131, out_scale=0.04),
    "grouped_tc_implicit": dict(n=2, h=12, w=13, cin=64, cout=64, k=3, groups=2, per_channel=True, out_scale=0.3, act=cases.enn.ACT_NONE),
    "grouped_tc_1x1_g4": dict(n=3, h=14, w=14, cin=64, cout=96, k=1, groups=4, w_zp=119, out_scale=0.03),
    "grouped_tc_1x1_g8_pc_relu": dict(n=2, h=20, w=20, cin=128, cout=128, k=1, groups=8, per_channel=True, out_scale=0.002, out_zp=0),
    "pointwise": dict(n=2, h=14, w=14, cin=96, cout=24, k=1, act=cases.enn.ACT_NONE),
    "per_channel": dict(n=2, h=14, w=14, cin=32, cout=48, k=3, per_channel=True, out_scale=0.3),
    "per_channel_1x1": dict(n=3, h=7, w=7, cin=160, cout=320, k=1, per_channel=True, out_scale=0.5, act=cases.enn.ACT_NONE),
    "relu": dict(n=1, h=8, w=8, cin=16, cout=16, k=3, act=cases.enn.ACT_RELU),
    "relu1": dict(n=1, h=8, w=8, cin=16, cout=16, k=3, act=cases.enn.ACT_RELU1, out_scale=0.01),
    "valid_pad": dict(n=1, h=10, w=11, cin=8, cout=8, k=3, pad="valid"),
    "asym_kernel": dict(n=1, h=9, w=12, cin=8, cout=8, kh=1, kw=5),
    "signed_act": dict(n=1, h=8, w=8, cin=8, cout=8, k=3, act_dtype=cases.enn.S8, in_zp=-3, out_zp=5, per_channel=True, out_scale=0.2),
    "big_multiplier": dict(n=1, h=6, w=6, cin=4, cout=4, k=1, in_scale=0.5, w_scale=0.5, out_scale=0.05, w_zp=3),
    "batch_stem_like": dict(n=2, h=32, w=32, cin=3, cout=32, k=3, stride=2, per_channel=True, out_scale=0.1),
    # implicit (tap-box) convolutions: swizzle spans 128 / 64 / 32, ragged grids, dilation, zero and non-zero input zero point
    "implicit_c128": dict(n=2, h=20, w=17, cin=128, cout=48, k=3),
    "implicit_c64_56": dict(n=2, h=56, w=56, cin=64, cout=64, k=3),
    "implicit_c32_dil": dict(n=1, h=19, w=23, cin=32, cout=16, k=3, dil=2),
    "implicit_zp0": dict(n=1, h=15, w=15, cin=64, cout=32, k=3, in_zp=0, per_channel=True, out_scale=0.4),
    "implicit_wide": dict(n=1, h=5, w=150, cin=32, cout=32, k=3),
    "implicit_5x5_valid": dict(n=1, h=12, w=12, cin=32, cout=24, k=5, pad="valid"),
    "implicit_c96": dict(n=1, h=9, w=9, cin=96, cout=40, k=3),
    # first-layer kernel (3x3 taps over 3 channels, >= 4096 output pixels): stride 2 per-channel, stride 1 with u8
    # per-tensor weights (row-sum correction), signed activations, VALID padding, odd widths (unaligned row starts)
    # ReLU-type outputs with multipliers from 0.03 to 3 (right shifts, e == 0, left shifts) in 1x1, implicit 3x3 and gathered form
    "relu_wide_mult_1x1": dict(n=2, h=14, w=14, cin=32, cout=48, k=1, per_channel=True, out_scale=0.0006, out_zp=0),
    "relu_wide_mult_3x3": dict(n=1, h=12, w=13, cin=32, cout=32, k=3, per_channel=True, out_scale=0.0006, act=cases.enn.ACT_RELU, out_zp=0),
    "relu_wide_mult_gather": dict(n=2, h=15, w=14, cin=8, cout=16, k=3, stride=2, per_channel=True, out_scale=0.0004, out_zp=0),
    "pack_1x1_c24_to_144_relu": dict(n=2, h=48, w=50, cin=24, cout=144, k=1, per_channel=True, out_scale=0.002, out_zp=0),
    "pack_1x1_c24_to_40_u8w": dict(n=1, h=64, w=66, cin=24, cout=40, k=1, w_zp=130, out_scale=0.03),
    "pack_1x1_c32_to_16": dict(n=2, h=48, w=50, cin=32, cout=16, k=1, per_channel=True, out_scale=0.3, act=cases.enn.ACT_NONE),
    "pack_1x1_c24_to_144_odd_rows": dict(n=1, h=65, w=65, cin=24, cout=144, k=1, per_channel=True, out_scale=0.002, out_zp=0),   # 4225 rows: no pixel pairs
    "pack_1x1_c40_to_64_pairs": dict(n=2, h=48, w=50, cin=40, cout=64, k=1, per_channel=True, out_scale=0.05, act=cases.enn.ACT_NONE),
    # rows of 96 / 144 / 192 bytes (not whole 128-byte lines), few output channels: the shapes of the MobileNetV2 project layers
    "pack_wide_1x1_c96_to_24": dict(n=2, h=48, w=50, cin=96, cout=24, k=1, per_channel=True, out_scale=0.4, act=cases.enn.ACT_NONE),
    "pack_wide_1x1_c144_to_32_u8w": dict(n=1, h=64, w=66, cin=144, cout=32, k=1, w_zp=130, out_scale=0.08, act=cases.enn.ACT_NONE),
    "pack_wide_1x1_c192_to_64_relu": dict(n=2, h=46, w=50, cin=192, cout=64, k=1, per_channel=True, out_scale=0.004, out_zp=0),
    # several M tiles per work unit requantised together: clamp = the whole byte (the saturating pack clamps), a clamp
    # below 255, a lower clamp above 0; M not a multiple of the unit; N = 96 (whole chunks) and N = 40
    "relu_sat_units_n96": dict(n=8, h=32, w=33, cin=16, cout=96, k=1, per_channel=True, out_scale=0.0235, out_zp=0),
    "relu_clamp120_units_n96": dict(n=8, h=32, w=33, cin=16, cout=96, k=1, per_channel=True, out_scale=0.05, out_zp=0),
    "relu_zp128_units_n96": dict(n=8, h=32, w=33, cin=16, cout=96, k=1, per_channel=True, out_scale=0.0235, out_zp=128),
    "relu_sat_units_n40": dict(n=5, h=31, w=33, cin=32, cout=40, k=1, per_channel=True, out_scale=0.0235, out_zp=0),
    "first_layer_s2": dict(n=4, h=66, w=71, cin=3, cout=32, k=3, stride=2, per_channel=True, out_scale=0.1),
    "first_layer_s1_u8w": dict(n=2, h=47, w=53, cin=3, cout=16, k=3, w_zp=121, out_scale=0.05),
    "first_layer_signed": dict(n=1, h=70, w=69, cin=3, cout=48, k=3, act_dtype=cases.enn.S8, in_zp=-7, out_zp=3, per_channel=True, out_scale=0.2),
    "first_layer_valid": dict(n=3, h=41, w=43, cin=3, cout=32, k=3, pad="valid", per_channel=True, out_scale=0.15, act=cases.enn.ACT_NONE),
    # signed activations with a negative lower clamp and outputs on both sides of zero (the packed epilogue adds the clamp
    # back per byte): in-place 1x1 with N a multiple of 16 and not, implicit 3x3, gathered, first layer, u8 weights
    "s8_none_1x1_n48": dict(n=2, h=14, w=14, cin=32, cout=48, k=1, act_dtype=cases.enn.S8, in_zp=-3, out_zp=-5, act=cases.enn.ACT_NONE, per_channel=True, out_scale=0.6),
    "s8_relu_zpm128_1x1_n40": dict(n=2, h=14, w=14, cin=32, cout=40, k=1, act_dtype=cases.enn.S8, in_zp=4, out_zp=-128, act=cases.enn.ACT_RELU, per_channel=True, out_scale=0.3),
    "s8_none_implicit_3x3": dict(n=1, h=12, w=13, cin=32, cout=32, k=3, act_dtype=cases.enn.S8, in_zp=-1, out_zp=7, act=cases.enn.ACT_NONE, per_channel=True, out_scale=1.5),
    "s8_relu6_zpm128_implicit": dict(n=2, h=9, w=9, cin=64, cout=24, k=3, act_dtype=cases.enn.S8, in_zp=0, out_zp=-128, per_channel=True, out_scale=0.03),
    "s8_none_gather_s2": dict(n=2, h=15, w=14, cin=8, cout=16, k=3, stride=2, act_dtype=cases.enn.S8, in_zp=-9, out_zp=0, act=cases.enn.ACT_NONE, per_channel=True, out_scale=0.5),
    "s8_none_first_layer": dict(n=1, h=70, w=69, cin=3, cout=32, k=3, act_dtype=cases.enn.S8, in_zp=-7, out_zp=-10, act=cases.enn.ACT_NONE, per_channel=True, out_scale=0.3),
    "s8_none_u8_weights": dict(n=2, h=10, w=10, cin=16, cout=32, k=1, act_dtype=cases.enn.S8, in_zp=5, out_zp=-3, act=cases.enn.ACT_NONE, w_zp=121, out_scale=0.08),
}


@pytest.mark.parametrize("name", list(CONV_CASES))
def test_conv2d_parity(enn, orc, ctx, name):
    d, x, w, b, sc = cases.conv_case(seed=_seed(name), **CONV_CASES[name])
    y_ref = orc.conv2d(d, x, w, b, sc)
    if name.startswith("s8_"):      # the case is only worth its name with outputs on both sides of zero
        assert (y_ref < 0).mean() > 0.02 and (y_ref >= 0).mean() > 0.02, ((y_ref < 0).mean(), name)
    op = enn.conv2d(ctx, d, w, b, sc)
    try:
        for impl in _impls(enn, op):
            op.set_impl(impl)
            _check(op, y_ref, x)
    finally:
        op.release()


def _sweep_params(seed):
    """One pseudo-random convolution / activation / quantisation combination (fixed by `seed`)."""
    rng = np.random.default_rng(1000 + seed)
    k = int(rng.choice([1, 1, 1, 3]))
    cin = int(rng.choice([3, 8, 16, 24, 32, 48, 64, 96]))
    cout = int(rng.choice([16, 24, 32, 48, 96, 144]))
    stride = int(rng.choice([1, 1, 2])) if k == 3 else 1
    per_channel = bool(rng.integers(0, 2))
    act = int(rng.choice([cases.enn.ACT_NONE, cases.enn.ACT_RELU, cases.enn.ACT_RELU6]))
    out_zp = int(rng.choice([0, 0, 5, 128])) if act != cases.enn.ACT_NONE else int(rng.integers(0, 256))
    h, w = int(rng.integers(33, 50)), int(rng.integers(33, 50))
    n = 4
    while (n * h * w) % 8:          # keep the row count divisible by every packing factor
        w += 1
    out_scale = float(np.exp(rng.uniform(np.log(3e-4), np.log(0.3))))
    kw = dict(n=n, h=h, w=w, cin=cin, cout=cout, k=k, stride=stride, per_channel=per_channel, act=act, out_zp=out_zp, out_scale=out_scale)
    if not per_channel:
        kw["w_zp"] = int(rng.integers(100, 156))
    return kw


@pytest.mark.parametrize("seed", range(24))
def test_conv2d_parity_sweep(enn, orc, ctx, seed):
    """Pseudo-random geometry x activation x quantisation combinations (>= 4096 output pixels, so that the packed,
    first-layer and ReLU-merged paths are all eligible) against the oracle, default implementation."""
    kw = _sweep_params(seed)
    d, x, w, b, sc = cases.conv_case(seed=seed, **kw)
    y_ref = orc.conv2d(d, x, w, b, sc)
    op = enn.conv2d(ctx, d, w, b, sc)
    try:
        _check(op, y_ref, x)
    finally:
        op.release()


def test_kat_perchannel_conv_gpu(enn, ctx):
    """Reference known-answer test gpu_userdriver_test.cc:474-575 through NCHW upload + layout conversion."""
    k = json.load(open(os.path.join(HERE, "golden", "kat_perchannel_conv.json")))
    n, c, h, w = k["input_dims_nchw"]
    x_nchw = np.array(k["input"], np.uint8)
    d = enn.conv_desc(n=n, h=h, w=w, cin=c, cout=3, kh=1, kw=1, per_channel=1, weight_dtype=enn.S8,
                      weight_layout=enn.W_OHWI, in_scale=k["input_scale"], in_zp=k["zero_point"],
                      out_scale=k["output_scale"], out_zp=k["zero_point"])
    op = enn.conv2d(ctx, d, np.array(k["weight"], np.int8), np.array(k["bias"], np.int32), np.array(k["scales"], np.float32))
    src = ctx.to_device(x_nchw)
    nhwc, out, out_nchw = ctx.malloc(6), ctx.malloc(9), ctx.malloc(9)
    ctx.check(enn.lib.enn_b200_nchw_to_nhwc(ctx.h, src, nhwc, n, c, h, w))
    op.execute(nhwc, out)
    ctx.check(enn.lib.enn_b200_nhwc_to_nchw(ctx.h, out, out_nchw, 1, 3, 3, 1))
    assert ctx.download(out_nchw, (9,)).tolist() == k["expect"]
    for p in (src, nhwc, out, out_nchw):
        ctx.free(p)
    op.release()


DW_CASES = {
    "config2_s1": dict(n=2),
    "config2_s2": dict(n=2, stride=2),
    "per_tensor": dict(n=1, h=17, w=19, c=24, per_channel=False, out_scale=0.08, out_zp=3),
    "multiplier2": dict(n=1, h=9, w=9, c=6, dm=2),
    "ohwi_5x5": dict(n=1, h=12, w=12, c=16, k=5, layout=cases.enn.W_OHWI),
    "odd_channels": dict(n=2, h=7, w=7, c=5),
    "dilated": dict(n=1, h=14, w=14, c=8, dil=2),
    "wide_c": dict(n=1, h=14, w=14, c=576),
    "c960_7x7": dict(n=2, h=7, w=7, c=960),
    "signed": dict(n=1, h=9, w=9, c=8, act_dtype=cases.enn.S8, in_zp=-5, out_zp=-128),
    "tiny": dict(n=1, h=1, w=1, c=4),
    "per_tensor_s2": dict(n=2, h=15, w=13, c=12, stride=2, per_channel=False, out_scale=0.08, out_zp=3),
    "relu_small_out_scale": dict(n=1, h=20, w=21, c=32, out_scale=0.004),           # multipliers up to 0.5: shifts down to e = 1
    "relu_s2_zp5": dict(n=2, h=21, w=20, c=48, stride=2, out_zp=5, out_scale=0.02),
    "s2_even": dict(n=1, h=16, w=16, c=8, stride=2),
    "ragged_rows": dict(n=3, h=10, w=6, c=4),
    "single_row": dict(n=1, h=1, w=9, c=8),
    "single_col": dict(n=1, h=9, w=1, c=8, stride=2),
    "relu": dict(n=1, h=8, w=8, c=8, act=cases.enn.ACT_RELU, out_zp=20),
    "none_act_zp128": dict(n=1, h=8, w=11, c=16, act=cases.enn.ACT_NONE, out_zp=128, out_scale=0.1),
    "tall": dict(n=1, h=70, w=5, c=4),
    # row-ring kernel (C % 16 == 0): several x tiles, ragged last strip, row ranges that cross image boundaries, one- and
    # two-row images, borders with a non-zero input zero point, both SAME-padding parities of stride 2, u8 weights
    "ring_c144_w56": dict(n=3, h=56, w=56, c=144),
    "ring_c144_s2_odd": dict(n=2, h=57, w=55, c=144, stride=2),
    "ring_c192_w28": dict(n=5, h=28, w=28, c=192, in_zp=3),
    "ring_c384_w14": dict(n=7, h=14, w=14, c=384),
    "ring_c576_s2": dict(n=3, h=14, w=14, c=576, stride=2, in_zp=0),
    "ring_c16_wide": dict(n=1, h=5, w=230, c=16),
    "ring_h1": dict(n=4, h=1, w=33, c=32),
    "ring_h2_s2": dict(n=4, h=2, w=9, c=64, stride=2),
    "ring_many_images": dict(n=40, h=7, w=10, c=32),
    "ring_many_images_s2": dict(n=37, h=9, w=11, c=48, stride=2, out_scale=0.02),
    "ring_per_tensor": dict(n=2, h=20, w=21, c=32, per_channel=False, out_scale=0.08, out_zp=3),
    "ring_per_tensor_s2_relu": dict(n=2, h=22, w=19, c=64, stride=2, per_channel=False, out_scale=0.03, out_zp=0),
    "ring_none_act": dict(n=2, h=13, w=17, c=96, act=cases.enn.ACT_NONE, out_zp=131, out_scale=0.1),
    # 225-256 channel quads: the eight-consumer-warp form of the ring kernel (one CTA per SM)
    "ring_big_c1024": dict(n=3, h=7, w=9, c=1024, in_zp=7),
    "ring_big_c912_s2": dict(n=5, h=14, w=14, c=912, stride=2),
    "ring_big_c960_none": dict(n=9, h=7, w=7, c=960, act=cases.enn.ACT_NONE, out_zp=128, out_scale=0.1),
    "beyond_ring_c1040": dict(n=2, h=7, w=7, c=1040),
    # output channels past cin * depth_multiplier: no filter, bias only (depthwise_conv_unequal)
    "unequal_pt": dict(n=2, h=9, w=10, c=6, dm=2, per_channel=False, out_scale=0.3, out_zp=90, act=cases.enn.ACT_NONE, extra_out=5),
    "unequal_pc_3x3_c32": dict(n=1, h=12, w=12, c=32, extra_out=16, out_scale=0.8, out_zp=100, act=cases.enn.ACT_NONE),
    "unequal_ohwi": dict(n=1, h=7, w=8, c=8, per_channel=False, layout=cases.enn.W_OHWI, extra_out=3, out_scale=0.3, out_zp=90, act=cases.enn.ACT_NONE),
}


@pytest.mark.parametrize("name", list(DW_CASES))
def test_depthwise_parity(enn, orc, ctx, name):
    d, x, w, b, sc = cases.depthwise_case(seed=_seed(name), **DW_CASES[name])
    y_ref = orc.depthwise(d, x, w, b, sc)
    op = enn.depthwise(ctx, d, w, b, sc)
    try:
        for impl in (enn.IMPL_DEPTHWISE, enn.IMPL_DIRECT):     # 3x3 fast path (when eligible) and general kernel
            op.set_impl(impl)
            _check(op, y_ref, x)
    finally:
        op.release()


@pytest.mark.parametrize("seed", range(16))
def test_depthwise_parity_sweep(enn, orc, ctx, seed):
    """Pseudo-random 3x3 depthwise layers (channels, stride, activation, zero points, output scale over three decades,
    so that right shifts down to 1 and both requantisation forms occur) against the oracle."""
    rng = np.random.default_rng(2000 + seed)
    act = int(rng.choice([cases.enn.ACT_NONE, cases.enn.ACT_RELU, cases.enn.ACT_RELU6]))
    kw = dict(n=2, h=int(rng.integers(9, 40)), w=int(rng.integers(9, 40)), c=int(rng.choice([4, 8, 12, 32, 48, 96, 144])),
              stride=int(rng.choice([1, 2])), per_channel=bool(rng.integers(0, 2)), act=act,
              out_zp=int(rng.choice([0, 0, 3, 128])) if act != cases.enn.ACT_NONE else int(rng.integers(0, 256)),
              out_scale=float(np.exp(rng.uniform(np.log(2e-3), np.log(0.2)))), in_zp=int(rng.choice([0, 17, 128])))
    if not kw["per_channel"]:
        kw["w_zp"] = int(rng.integers(100, 156))
    d, x, w, b, sc = cases.depthwise_case(seed=seed, **kw)
    y_ref = orc.depthwise(d, x, w, b, sc)
    op = enn.depthwise(ctx, d, w, b, sc)
    try:
        _check(op, y_ref, x)
    finally:
        op.release()


@pytest.mark.parametrize("seed", range(12))
def test_fc_parity_sweep(enn, orc, ctx, seed):
    """Pseudo-random FullyConnected shapes (packed, narrow-span, GEMV and plain paths) x activation x quantisation."""
    rng = np.random.default_rng(3000 + seed)
    act = int(rng.choice([cases.enn.ACT_NONE, cases.enn.ACT_RELU, cases.enn.ACT_RELU6]))
    kw = dict(m=int(rng.choice([3, 8, 200, 4104, 4112])), k=int(rng.choice([16, 32, 48, 64, 96, 160, 512])),
              n=int(rng.choice([16, 24, 40, 96, 272])), per_channel=bool(rng.integers(0, 2)), act=act,
              out_zp=int(rng.choice([0, 0, 9, 128])) if act != cases.enn.ACT_NONE else int(rng.integers(0, 256)))
    kw["out_scale"] = cases.fc_out_scale(kw["k"]) * float(np.exp(rng.uniform(np.log(0.02), np.log(2.0))))
    if not kw["per_channel"]:
        kw["w_zp"] = int(rng.integers(100, 156))
    d, x, w, b, sc = cases.fc_case(seed=seed, **kw)
    y_ref = orc.fully_connected(d, x, w, b, sc)
    op = enn.fully_connected(ctx, d, w, b, sc)
    try:
        _check(op, y_ref, x)
    finally:
        op.release()


@pytest.mark.parametrize("name", ["config2_s1", "config2_s2", "wide_c", "ring_c144_s2_odd", "none_act_zp128", "ring_per_tensor"])
def test_depthwise_register_streamed_kernel(enn, orc, name):
    """The register-streamed 3x3 kernel (what channel counts that are not a multiple of 16, or more than 896, use) on
    shapes the row-ring kernel normally takes, selected with the planner option `dw_legacy`."""
    c2 = enn.Context(0)
    try:
        c2.set_option("dw_legacy", 1)
        d, x, w, b, sc = cases.depthwise_case(seed=_seed(name), **DW_CASES[name])
        op = enn.depthwise(c2, d, w, b, sc)
        try:
            _check(op, orc.depthwise(d, x, w, b, sc), x)
        finally:
            op.release()
    finally:
        c2.close()


def test_depthwise_unaligned_pointers(enn, orc, ctx):
    """Device pointers at odd offsets (sub-buffers): the 16-byte and 4-byte aligned fast paths step aside."""
    d, x, w, b, sc = cases.depthwise_case(seed=11, n=2, h=12, w=13, c=32)
    y_ref = orc.depthwise(d, x, w, b, sc).reshape(-1)
    op = enn.depthwise(ctx, d, w, b, sc)
    buf_in, buf_out = ctx.malloc(x.nbytes + 64), ctx.malloc(y_ref.size + 64)
    try:
        for off_in, off_out in ((1, 0), (4, 0), (0, 3), (5, 7), (16, 4)):
            pin = type(buf_in)(buf_in.value + off_in)
            pout = type(buf_out)(buf_out.value + off_out)
            ctx.upload(pin, x)
            op.execute(pin, pout)
            assert np.array_equal(ctx.download(pout, (y_ref.size,)), y_ref), (off_in, off_out)
    finally:
        ctx.free(buf_in)
        ctx.free(buf_out)
        op.release()


DECONV_CASES = {
    "config4_small": dict(n=1, h=16, w=16),
    "ohwi": dict(n=2, h=6, w=5, cin=16, cout=8, layout=cases.enn.W_OHWI),
    "per_channel": dict(n=1, h=8, w=8, cin=32, cout=16, per_channel=True, out_scale=0.5),
    "k3_s2": dict(n=1, h=7, w=7, cin=8, cout=8, k=3, stride=2, pad=0),
    "k2_s2": dict(n=1, h=7, w=9, cin=8, cout=4, k=2, stride=2, pad=0),
    "s1": dict(n=1, h=6, w=6, cin=8, cout=8, k=3, stride=1, pad=1),
    "relu6": dict(n=1, h=5, w=5, cin=4, cout=4, act=cases.enn.ACT_RELU6),
    "implicit_config4_small": dict(n=2, h=16, w=16, cin=128, cout=64),
    "implicit_c32_k3": dict(n=1, h=9, w=7, cin=32, cout=16, k=3, stride=2, pad=0),
    "implicit_c64_s3": dict(n=1, h=6, w=6, cin=64, cout=16, k=4, stride=3, pad=1),
    "s8_none_implicit": dict(n=2, h=8, w=8, cin=32, cout=16, per_channel=True, out_scale=1.2, act_dtype=cases.enn.S8, in_zp=-4, out_zp=-6),
    "s8_relu_zpm128_u8w": dict(n=1, h=7, w=9, cin=16, cout=24, act_dtype=cases.enn.S8, in_zp=3, out_zp=-128, act=cases.enn.ACT_RELU, out_scale=0.1),
}


@pytest.mark.parametrize("name", list(DECONV_CASES))
def test_deconv_parity(enn, orc, ctx, name):
    d, x, w, b, sc = cases.deconv_case(seed=_seed(name), **DECONV_CASES[name])
    y_ref = orc.deconv(d, x, w, b, sc)
    op = enn.deconv(ctx, d, w, b, sc)
    try:
        for impl in _impls(enn, op):
            op.set_impl(impl)
            _check(op, y_ref, x)
    finally:
        op.release()


FC_CASES = {
    "gemv": dict(m=1, k=512, n=256),
    "small": dict(m=4, k=256, n=64),
    "mid": dict(m=256, k=1024, n=1024),
    "ragged": dict(m=37, k=100, n=29),
    "per_tensor": dict(m=8, k=128, n=64, per_channel=False),
    "relu6": dict(m=8, k=128, n=64, act=cases.enn.ACT_RELU6),
    "fc1000": dict(m=200, k=1280, n=1000),
    "big_k": dict(m=130, k=4096, n=272),
    "per_tensor_wide": dict(m=300, k=256, n=520, per_channel=False),
    "per_tensor_zp128": dict(m=129, k=64, n=48, per_channel=False, w_zp=128),
    "k16_n16": dict(m=1000, k=16, n=16),
    "mixed_shift": dict(m=150, k=64, n=80, out_scale=0.0015),      # multipliers 0.013 .. 1.33: e >= 1, e == 0 and left shifts
    "mixed_shift_per_tensor": dict(m=150, k=32, n=40, per_channel=False, w_scale=0.05, out_scale=0.0012),
    "n24": dict(m=300, k=96, n=24),
    "gemv_m1_k4096": dict(m=1, k=4096, n=1000),
    "gemv_m3_per_tensor": dict(m=3, k=1280, n=77, per_channel=False),
    "gemv_m8_mixed_shift": dict(m=8, k=64, n=80, out_scale=0.0015),
    # ReLU-type outputs (lower clamp == output zero point: merged 64-bit epilogue) across right shifts, e == 0 and left shifts
    "relu_mixed_shift": dict(m=150, k=64, n=80, out_scale=0.0015, act=cases.enn.ACT_RELU, out_zp=0),
    "relu6_mixed_shift_zp7": dict(m=260, k=160, n=144, out_scale=0.003, act=cases.enn.ACT_RELU6, out_zp=7),
    "relu_per_tensor_mixed": dict(m=150, k=32, n=48, per_channel=False, w_scale=0.05, out_scale=0.0012, act=cases.enn.ACT_RELU, out_zp=0),
    "relu_small_mult": dict(m=300, k=96, n=96, act=cases.enn.ACT_RELU6, out_zp=0),
    # pixel packing (K of 16 / 32 / 64 bytes, few output channels, >= 4096 rows): block-diagonal weights, f rows per 128-byte line
    "pack_k32_n16": dict(m=4104, k=32, n=16),
    "pack_k16_n24_per_tensor": dict(m=4104, k=16, n=24, per_channel=False, w_zp=119),
    "pack_k64_n96_relu": dict(m=4098, k=64, n=96, act=cases.enn.ACT_RELU, out_zp=0, out_scale=0.004),
    "pack_k32_n48_mixed_shift": dict(m=4100, k=32, n=48, out_scale=0.0012),
    # several M tiles requantised together per column: 3 tiles per unit taken 2 at a time (row-sum column, u8 weights),
    # 4 at a time with a last unit of 3 tiles and a ragged last tile, 2 at a time with two N tiles
    "group3_rowsum_k128_n64": dict(m=120000, k=128, n=64, per_channel=False, w_zp=119),
    "group4_ragged_k128_n64": dict(m=128 * 4 * 300 + 128 * 2 + 5, k=128, n=64),
    "group2_two_n_tiles_k256_n256_relu": dict(m=40000, k=256, n=256, act=cases.enn.ACT_RELU6, out_zp=0, out_scale=0.01),
    # one k-block and more than 128 output channels: tiles of at most 128 columns, two M tiles per accumulator buffer;
    # whole and ragged column counts, a half-empty last N tile, general and ReLU-type epilogues, signed activations,
    # and u8 weights (row-sum column: the rule does not apply)
    "narrow_n_k32_n192_relu": dict(m=3000, k=32, n=192, act=cases.enn.ACT_RELU6, out_zp=0, out_scale=0.01),
    "narrow_n_k64_n200_none": dict(m=1000, k=64, n=200, act=cases.enn.ACT_NONE),
    "narrow_n_k96_n576_relu": dict(m=2000, k=96, n=576, act=cases.enn.ACT_RELU, out_zp=0, out_scale=0.02),
    "narrow_n_k128_n130_s8": dict(m=700, k=128, n=130, act_dtype=cases.enn.S8, in_zp=-3, out_zp=-7),
    "narrow_n_k16_n144_ragged_m": dict(m=4097, k=16, n=144, act=cases.enn.ACT_RELU6, out_zp=0, out_scale=0.01),
    "narrow_n_k32_n192_u8w": dict(m=1500, k=32, n=192, per_channel=False, w_zp=119),
    "pack_wide_k96_n24": dict(m=4104, k=96, n=24, act=cases.enn.ACT_NONE),
    "pack_wide_k144_n24_per_tensor": dict(m=4100, k=144, n=24, per_channel=False, w_zp=119, act=cases.enn.ACT_NONE),
    "pack_wide_k192_n32": dict(m=4098, k=192, n=32, act=cases.enn.ACT_NONE, out_scale=0.3),
    # signed activations, negative lower clamp, outputs on both sides of zero
    "s8_none_n64": dict(m=300, k=256, n=64, act_dtype=cases.enn.S8, in_zp=-5, out_zp=3),
    "s8_none_n29_gemv": dict(m=5, k=128, n=29, act_dtype=cases.enn.S8, in_zp=6, out_zp=-20),
    "s8_relu_zpm128_n40": dict(m=200, k=96, n=40, act_dtype=cases.enn.S8, in_zp=0, out_zp=-128, act=cases.enn.ACT_RELU),
    "s8_none_pack_k32_n16": dict(m=4104, k=32, n=16, act_dtype=cases.enn.S8, in_zp=-2, out_zp=1),
}


@pytest.mark.parametrize("name", list(FC_CASES))
def test_fc_parity(enn, orc, ctx, name):
    d, x, w, b, sc = cases.fc_case(seed=_seed(name), **FC_CASES[name])
    y_ref = orc.fully_connected(d, x, w, b, sc)
    op = enn.fully_connected(ctx, d, w, b, sc)
    try:
        for impl in _impls(enn, op):
            op.set_impl(impl)
            _check(op, y_ref, x)
    finally:
        op.release()


def _sub_batch(d, x, idx):
    """Descriptor and input restricted to the images `idx` of the batch (for the oracle on sampled images)."""
    ds = type(d).from_buffer_copy(d)
    ds.n = len(idx)
    return ds, np.ascontiguousarray(x[idx])


@pytest.mark.parametrize("stride", [1, 2])
def test_depthwise_config2_benchmark_size(enn, orc, ctx, stride):
    """Benchmark configuration 2 at its full size (64 x 112 x 112 x 32): first, middle and last images against the oracle,
    and every image against the first (all 64 are computed independently from a repeated input)."""
    d, x, w, b, sc = cases.depthwise_case(seed=0, n=64, stride=stride)
    op = enn.depthwise(ctx, d, w, b, sc)
    try:
        y = op.run(x).reshape(op.out_shape)
        idx = [0, 31, 63]
        ds, xs = _sub_batch(d, x, idx)
        assert np.array_equal(y[idx], orc.depthwise(ds, xs, w, b, sc))
        x_rep = np.ascontiguousarray(np.broadcast_to(x[5], x.shape))
        y_rep = op.run(x_rep).reshape(op.out_shape)
        assert np.array_equal(y_rep, np.broadcast_to(y[5], y.shape))
    finally:
        op.release()


def test_deconv_config4_benchmark_size(enn, orc, ctx):
    """Benchmark configuration 4 at its full size (8 x 64 x 64 x 128 -> 8 x 128 x 128 x 64): first and last images
    against the oracle, every image against image 3 on a repeated input."""
    d, x, w, b, sc = cases.deconv_case(seed=0, n=8, h=64, w=64)
    op = enn.deconv(ctx, d, w, b, sc)
    try:
        y = op.run(x).reshape(op.out_shape)
        idx = [0, 7]
        ds, xs = _sub_batch(d, x, idx)
        assert np.array_equal(y[idx], orc.deconv(ds, xs, w, b, sc))
        x_rep = np.ascontiguousarray(np.broadcast_to(x[3], x.shape))
        y_rep = op.run(x_rep).reshape(op.out_shape)
        assert np.array_equal(y_rep, np.broadcast_to(y[3], y.shape))
    finally:
        op.release()


def test_conv_config1_batched_benchmark_size(enn, orc, ctx):
    """Configuration 1 (per-tensor u8 3x3 convolution, 56 x 56 x 64) at batch 1 whole and at batch 256 on sampled images."""
    d, x, w, b, sc = cases.conv_case(seed=0)
    op = enn.conv2d(ctx, d, w, b, sc)
    try:
        assert np.array_equal(op.run(x).reshape(op.out_shape), orc.conv2d(d, x, w, b, sc))
    finally:
        op.release()
    d, x, w, b, sc = cases.conv_case(seed=0, n=256)
    op = enn.conv2d(ctx, d, w, b, sc)
    try:
        y = op.run(x).reshape(op.out_shape)
        idx = [0, 128, 255]
        ds, xs = _sub_batch(d, x, idx)
        assert np.array_equal(y[idx], orc.conv2d(ds, xs, w, b, sc))
    finally:
        op.release()


def test_fc_config3_gemv_benchmark_size(enn, orc, ctx):
    """Benchmark configuration 3, M = 1 (1 x 4096 x 4096): every output against the oracle."""
    d, x, w, b, sc = cases.fc_case(seed=0, m=1, k=4096, n=4096)
    op = enn.fully_connected(ctx, d, w, b, sc)
    try:
        assert op.info.impl == enn.IMPL_GEMV
        assert np.array_equal(op.run(x).reshape(1, 4096), orc.fully_connected(d, x, w, b, sc))
    finally:
        op.release()


def test_fc_full_size_sampled_rows(enn, orc, ctx):
    """4096 x 4096 x 4096 (the largest benchmark GEMM): rows sampled across all M tiles against the oracle."""
    d, x, w, b, sc = cases.fc_case(seed=5, m=4096, k=4096, n=4096)
    op = enn.fully_connected(ctx, d, w, b, sc)
    try:
        y = op.run(x).reshape(4096, 4096)
        rows = np.r_[0:4, 127:130, 2047:2050, 4092:4096, np.random.default_rng(0).integers(0, 4096, 18)]
        ds = type(d).from_buffer_copy(d)
        ds.m = len(rows)
        y_ref = orc.fully_connected(ds, np.ascontiguousarray(x[rows]), w, b, sc)
        assert np.array_equal(y[rows], y_ref)
        assert len(np.unique(y)) > 100          # outputs are not saturated
    finally:
        op.release()


@pytest.mark.parametrize("m,k,n,w_zp", [(4096, 4096, 4096, None), (4230, 1024, 2500, 131)])
def test_fc_cta_pair_mode(enn, orc, m, k, n, w_zp):
    """The opt-in CTA-pair (cta_group::2) GEMM: same bytes as the oracle on sampled rows; the second shape has an odd
    number of M tiles (the last pair's second half lies outside the matrix), ragged N and the row-sum correction."""
    ctx = enn.Context(0)
    ctx.set_option("tc_pair", 1)
    kw = {} if w_zp is None else dict(w_zp=w_zp, per_channel=False)     # per-tensor u8 weights: zw' != 0
    d, x, w, b, sc = cases.fc_case(seed=9, m=m, k=k, n=n, **kw)
    op = enn.fully_connected(ctx, d, w, b, sc)
    try:
        assert op.info.impl == enn.IMPL_TCGEN05
        y = op.run(x).reshape(m, n)
        rows = np.r_[0:3, 126:131, 255:258, m - 260:m - 254, m - 3:m, np.random.default_rng(1).integers(0, m, 12)]
        ds = type(d).from_buffer_copy(d)
        ds.m = len(rows)
        y_ref = orc.fully_connected(ds, np.ascontiguousarray(x[rows]), w, b, sc)
        assert np.array_equal(y[rows], y_ref)
    finally:
        op.release()
        ctx.close()


@pytest.mark.parametrize("count,act", [(1, 0), (15, 0), (4097, 3), (1 << 20, 0), (56 * 56 * 24 * 3, 0)])
def test_add_parity(enn, orc, ctx, count, act):
    rng = np.random.default_rng(count)
    a = rng.integers(0, 256, count, dtype=np.int64).astype(np.uint8)
    b = rng.integers(0, 256, count, dtype=np.int64).astype(np.uint8)
    d = enn.AddDesc(count=count, activation=act, act_dtype=enn.U8, in0_scale=0.031, in0_zp=120, in1_scale=0.047,
                    in1_zp=131, out_scale=0.06, out_zp=126)
    op = enn.add(ctx, d)
    try:
        _check(op, orc.add(d, a, b), a, b)
    finally:
        op.release()


# four-channels-per-thread kernel: padded windows (ragged at the borders), signed bytes, a clamp that bites
@pytest.mark.parametrize("shape", [(2, 9, 10, 24, 3, 2, 1, "u8", 0), (2, 7, 7, 64, 7, 1, 0, "s8", 0), (3, 8, 8, 12, 3, 1, 1, "s8", 1),
                                   (1, 12, 12, 8, 5, 3, 2, "u8", 3)])
def test_avgpool_vec4_parity(enn, orc, ctx, shape):
    n, h, w, c, k, s, pad, dt, act = shape
    rng = np.random.default_rng(h * w + c)
    signed = dt == "s8"
    x = rng.integers(-128 if signed else 0, 128 if signed else 256, (n, h, w, c), dtype=np.int64).astype(np.int8 if signed else np.uint8)
    oh, ow = (h + 2 * pad - k) // s + 1, (w + 2 * pad - k) // s + 1
    d = enn.PoolDesc(n=n, h=h, w=w, c=c, kh=k, kw=k, stride_h=s, stride_w=s, pad_t=pad, pad_l=pad, out_h=oh, out_w=ow,
                     activation=act, act_dtype=enn.S8 if signed else enn.U8, out_scale=0.5, out_zp=-3 if signed else 100)
    op = enn.avgpool(ctx, d)
    try:
        _check(op, orc.avgpool(d, x), x)
    finally:
        op.release()


# pair-table kernel (>= 2^20 elements): a tail after the 16-byte groups, a clamp that bites, signed bytes, flat inputs
@pytest.mark.parametrize("count,act,dt,flat", [((1 << 21) + 5, 3, "u8", False), ((1 << 20) + 16, 0, "s8", False),
                                               (1 << 20, 1, "u8", True)])
def test_add_pair_table_parity(enn, orc, ctx, count, act, dt, flat):
    rng = np.random.default_rng(count + act)
    signed = dt == "s8"
    lo, hi, npdt = (-128, 128, np.int8) if signed else (0, 256, np.uint8)
    a = rng.integers(lo, hi, count, dtype=np.int64).astype(npdt)
    b = rng.integers(lo, hi, count, dtype=np.int64).astype(npdt)
    if flat:
        b[:] = 131
    d = enn.AddDesc(count=count, activation=act, act_dtype=enn.S8 if signed else enn.U8, in0_scale=0.031,
                    in0_zp=-8 if signed else 120, in1_scale=0.047, in1_zp=3 if signed else 131, out_scale=0.06,
                    out_zp=-2 if signed else 126)
    op = enn.add(ctx, d)
    try:
        _check(op, orc.add(d, a, b), a, b)
    finally:
        op.release()


@pytest.mark.parametrize("shape", [(2, 7, 7, 1280, 7, 1), (1, 9, 9, 16, 3, 2), (3, 5, 6, 7, 2, 2)])
def test_avgpool_parity(enn, orc, ctx, shape):
    n, h, w, c, k, s = shape
    rng = np.random.default_rng(h * w)
    x = rng.integers(0, 256, (n, h, w, c), dtype=np.int64).astype(np.uint8)
    oh, ow = (h - k) // s + 1, (w - k) // s + 1
    d = enn.PoolDesc(n=n, h=h, w=w, c=c, kh=k, kw=k, stride_h=s, stride_w=s, pad_t=0, pad_l=0, out_h=oh, out_w=ow,
                     activation=0, act_dtype=enn.U8, out_scale=0.02, out_zp=0)
    op = enn.avgpool(ctx, d)
    try:
        _check(op, orc.avgpool(d, x), x)
    finally:
        op.release()


def test_bounded_wait_gives_up_and_reports(enn, orc, ctx):
    """Failure detection on the device without a fault: one execute of a tensor-core operator is starved of its operand
    copies (nothing is issued, the wait limit is a fraction of a millisecond), the kernel gives up with nothing in
    flight, frees its tensor memory and returns; the host then reads the code, the operator refuses to run until the
    error is cleared, and afterwards it (and a freshly prepared one) computes the right bytes again."""
    d, x, w, b, sc = cases.conv_case(seed=5, n=2, h=16, w=16, cin=64, cout=64, k=1, per_channel=True, out_scale=0.3)
    y_ref = orc.conv2d(d, x, w, b, sc).reshape(-1)
    op = enn.conv2d(ctx, d, w, b, sc)
    try:
        assert op.info.impl == enn.IMPL_TCGEN05
        assert np.array_equal(op.run(x), y_ref)
        op.test_starve_next()
        op.run(x)                                   # the starved launch itself is enqueued without an error
        ctx.sync()
        with pytest.raises(enn.EnnError) as e:
            op.run(x)
        assert e.value.status == enn.CUDA_FAILURE and "barrier wait" in str(e.value)
        op.clear_error()
        assert np.array_equal(op.run(x), y_ref)
        op2 = enn.conv2d(ctx, d, w, b, sc)
        assert np.array_equal(op2.run(x), y_ref)
        op2.release()
    finally:
        op.release()


def test_options_and_limits(enn, ctx):
    c2 = enn.Context(0)
    try:
        with pytest.raises(enn.EnnError):
            c2.set_option("no_such_option", 1)
        with pytest.raises(enn.EnnError):
            c2.set_option("tc_bn", 64)              # narrower tiles than the epilogue supports are refused
        c2.set_option("no_gemv", 1)
        with pytest.raises(enn.EnnError):
            c2.mma_peak(0, 256, 1 << 20)            # would keep every SM busy for a long time
    finally:
        c2.close()


def _rebind_check(enn, orc, ctx, prepare, oracle, d, x, w, b, sc, dyn_w, dyn_b, rounds=2):
    """Operators whose filter / bias are runtime tensors: every rebind takes the tensors' current device contents."""
    d.weights_as_input, d.bias_as_input = int(dyn_w), int(dyn_b)
    op = prepare(ctx, d, None if dyn_w else w, None if dyn_b else b, sc)
    wd, bd = ctx.to_device(w), ctx.to_device(b)
    xd = ctx.to_device(x)
    od = ctx.malloc(op.info.out_bytes)
    try:
        with pytest.raises(enn.EnnError) as e:
            op.execute(xd, od)                      # nothing bound yet
        assert e.value.status == enn.FAILURE
        rng = np.random.default_rng(11)
        for r in range(rounds):
            if r:                                   # new contents in the same device buffers
                if dyn_w:
                    w = rng.integers(np.iinfo(w.dtype).min, int(np.iinfo(w.dtype).max) + 1, w.shape, dtype=np.int64).astype(w.dtype)
                    ctx.upload(wd, w)
                if dyn_b:
                    b = (b + rng.integers(-300, 300, b.shape)).astype(np.int32)
                    ctx.upload(bd, b)
            op.rebind_constants(wd if dyn_w else None, bd if dyn_b else None)
            op.execute(xd, od)
            ctx.sync()
            y = ctx.download(od, (op.info.out_bytes,), np.uint8)
            d.weights_as_input = d.bias_as_input = 0
            y_ref = oracle(d, x, w, b, sc)
            assert np.array_equal(y, y_ref.view(np.uint8).reshape(-1)), f"round {r}"
    finally:
        for p_ in (wd, bd, xd, od):
            ctx.free(p_)
        op.release()


@pytest.mark.parametrize("dyn_w,dyn_b", [(True, True), (True, False), (False, True)])
def test_runtime_filter_and_bias_conv(enn, orc, ctx, dyn_w, dyn_b):
    # CLConvolution.cpp:75-76, CLGEMMConvolutionQuantized.cpp:142-160: filter / bias that are not constant tensors
    d, x, w, b, sc = cases.conv_case(seed=_seed("dynconv"), n=2, h=20, w=20, cin=32, cout=48, per_channel=False)
    _rebind_check(enn, orc, ctx, enn.conv2d, orc.conv2d, d, x, w, b, sc, dyn_w, dyn_b)


def test_runtime_filter_depthwise_fc_deconv(enn, orc, ctx):
    d, x, w, b, sc = cases.depthwise_case(seed=_seed("dyndw"), n=1, h=24, w=24, c=32, per_channel=True)
    _rebind_check(enn, orc, ctx, enn.depthwise, orc.depthwise, d, x, w, b, sc, True, True)
    d, x, w, b, sc = cases.fc_case(seed=_seed("dynfc"), m=8, k=256, n=64, per_channel=False, w_zp=119)
    _rebind_check(enn, orc, ctx, enn.fully_connected, orc.fully_connected, d, x, w, b, sc, True, False)
    d, x, w, b, sc = cases.deconv_case(seed=_seed("dyndc"), n=1, h=8, w=8, cin=32, cout=16)
    _rebind_check(enn, orc, ctx, enn.deconv, orc.deconv, d, x, w, b, sc, True, True)


def test_runtime_constants_limits(enn, ctx):
    d, x, w, b, sc = cases.conv_case(seed=3, h=8, w=8, cin=8, cout=8)
    op = enn.conv2d(ctx, d, w, b, sc)
    with pytest.raises(enn.EnnError):
        op.rebind_constants(None, None)             # prepared with constant tensors
    op.release()
    d.weights_as_input = 1
    with pytest.raises(enn.EnnError):
        enn.conv2d(ctx, d, w, None, sc)             # the bias is still a constant and must be given
    op = enn.conv2d(ctx, d, None, b, sc)
    with pytest.raises(enn.EnnError):
        op.rebind_constants(None, None)             # the flagged tensor is missing
    ol = enn.OpList(ctx)
    t0, t1 = ol.tensor(x.nbytes), ol.tensor(op.info.out_bytes)
    with pytest.raises(enn.EnnError):
        ol.add(op, [t0], t1)                        # a captured launch sequence would hold stale constants
    ol.destroy()
    op.release()


FUSED_ADD_CASES = {
    # name: (conv case, add is (conv, other) or (other, conv)); shapes of the MobileNetV2 project layers and their tiling modes
    "project_56x56_144_to_24_packed": (dict(n=64, h=56, w=56, cin=144, cout=24, k=1, per_channel=True, out_scale=0.3, act=0, out_zp=128), False),
    "project_14x14_384_to_64": (dict(n=6, h=14, w=14, cin=384, cout=64, k=1, per_channel=True, out_scale=0.3, act=0, out_zp=121), True),
    "project_7x7_960_to_160": (dict(n=9, h=7, w=7, cin=960, cout=160, k=1, per_channel=True, out_scale=0.25, act=0, out_zp=130), False),
    "u8_weights_partial_tile": (dict(n=1, h=19, w=21, cin=64, cout=48, k=1, w_zp=131, out_scale=0.06, act=0, out_zp=119), False),
    "implicit_3x3": (dict(n=2, h=12, w=13, cin=32, cout=32, k=3, per_channel=True, out_scale=0.5, act=0, out_zp=125), True),
}


@pytest.mark.parametrize("name", list(FUSED_ADD_CASES))
def test_conv_with_fused_add(enn, orc, ctx, name):
    """CONV_2D -> ADD with the add in the convolution's epilogue equals the two operators run one after the other."""
    kw, conv_second = FUSED_ADD_CASES[name]
    d, x, w, b, sc = cases.conv_case(seed=_seed("fadd_" + name), **kw)
    y_conv = orc.conv2d(d, x, w, b, sc)
    rng = np.random.default_rng(_seed("fadd_res_" + name))
    res = rng.integers(0, 256, y_conv.shape, dtype=np.int64).astype(np.uint8)
    ad = enn.AddDesc(count=y_conv.size, activation=0, act_dtype=enn.U8, in0_scale=0.031, in0_zp=120, in1_scale=0.047, in1_zp=131,
                     out_scale=0.06, out_zp=126)
    y_ref = orc.add(ad, res, y_conv) if conv_second else orc.add(ad, y_conv, res)
    op = enn.conv2d(ctx, d, w, b, sc)
    addop = enn.add(ctx, ad)
    op.fuse_add(addop, conv_second)
    xd, rd = ctx.to_device(x), ctx.to_device(res)
    od = ctx.malloc(y_ref.size)
    try:
        with pytest.raises(enn.EnnError):
            op.execute(xd, od)                      # the second addend is missing
        op.execute2(xd, rd, od)
        ctx.sync()
        y = ctx.download(od, y_ref.shape, np.uint8)
        assert np.array_equal(y, y_ref), f"{(y != y_ref).sum()} of {y.size} differ"
        op.execute2(xd, rd, rd)                     # in place over the other addend (what an operator list may do)
        ctx.sync()
        assert np.array_equal(ctx.download(rd, y_ref.shape, np.uint8), y_ref)
    finally:
        for p_ in (xd, rd, od):
            ctx.free(p_)
        op.release()


def test_fused_add_refusals(enn, ctx):
    d, x, w, b, sc = cases.conv_case(seed=5, n=2, h=14, w=14, cin=32, cout=48, k=1, per_channel=True, out_scale=0.0235, out_zp=0)   # ReLU6: merged epilogue
    op = enn.conv2d(ctx, d, w, b, sc)
    ad = enn.AddDesc(count=op.info.out_bytes, activation=0, act_dtype=enn.U8, in0_scale=0.03, in0_zp=0, in1_scale=0.04, in1_zp=3, out_scale=0.06, out_zp=1)
    addop = enn.add(ctx, ad)
    with pytest.raises(enn.EnnError):
        op.fuse_add(addop)
    y = op.run(x)                                   # both operators are still usable
    assert y.size == op.info.out_bytes
    ad.count += 16
    other = enn.add(ctx, ad)
    with pytest.raises(enn.EnnError):
        op.fuse_add(other)                          # not an add over this convolution's output
    for o in (op, addop, other):
        o.release()


def test_oplist_profile_and_nodes(enn, ctx):
    """Per-operator device times of a list (the per-operator bracket the reference's executor puts around every op)."""
    import importlib
    mn = importlib.import_module(enn.__name__ + ".mobilenet")
    layers, _ = mn.build_model(seed=0, calib_images=1)
    ol, info = mn.make_oplist(enn, ctx, layers, 8)
    try:
        nodes = ol.nodes()
        n_add = sum(1 for L in layers if L["kind"] == "add")
        fused = sum(1 for (_, kind, nin) in nodes if kind == 0 and nin == 2)
        assert len(nodes) == len(layers) - fused and 0 < fused <= n_add      # at 8 images every add is small enough to fuse
        assert ol.stats()["kernel_launches"] == sum(i.kernel_launches for (i, _, _) in nodes)
        us = ol.profile(3)
        assert len(us) == len(nodes) and all(0.5 < t < 5000 for t in us), us
        with pytest.raises(enn.EnnError):
            ol.ctx.check(enn.lib.enn_b200_oplist_profile(ol.h, 0, None, 0))      # no repeats, no buffer
    finally:
        ol.destroy()


def test_grouped_conv_runs_on_tensor_cores(enn, ctx):
    d, x, w, b, sc = cases.conv_case(seed=9, n=2, h=14, w=14, cin=64, cout=96, k=1, groups=4)
    op = enn.conv2d(ctx, d, w, b, sc)
    assert op.info.impl == enn.IMPL_TCGEN05
    op.release()
    c2 = enn.Context(0)
    try:
        c2.set_option("no_grouped_tc", 1)
        op = enn.conv2d(c2, d, w, b, sc)
        assert op.info.impl == enn.IMPL_DIRECT
        op.release()
    finally:
        c2.close()


def test_error_paths(enn, ctx):
    d, x, w, b, sc = cases.conv_case(h=4, w=4, cin=4, cout=4)
    d.cin = 0
    with pytest.raises(enn.EnnError) as e:
        enn.conv2d(ctx, d, w, b, sc)
    assert e.value.status == enn.INVALID_PARAMS
    d, x, w, b, sc = cases.conv_case(h=4, w=4, cin=4, cout=4, per_channel=True)
    with pytest.raises(enn.EnnError):
        enn.conv2d(ctx, d, w, b, None)          # per-channel without scales
    d, x, w, b, sc = cases.conv_case(h=4, w=4, cin=6, cout=4, groups=4)
    with pytest.raises(enn.EnnError):
        enn.conv2d(ctx, d, w, b, sc)            # channels not divisible by groups
    d, x, w, b, sc = cases.conv_case(h=4, w=4, cin=4, cout=4)
    op = enn.conv2d(ctx, d, w, b, sc)
    with pytest.raises(enn.EnnError):
        op.execute(None, None)
    op.release()


def test_bias_scale_mismatch_gpu(enn, orc, ctx):
    d, x, w, b, sc = cases.conv_case(seed=1, h=6, w=6, cin=4, cout=4, act=enn.ACT_NONE)
    d.bias_scale = 0.5
    op = enn.conv2d(ctx, d, w, b, sc)
    y = op.run(x)
    assert np.all(y == d.out_zp)
    op.release()


def test_oplist_mobilenet_small(enn, orc, ctx):
    """Whole MobileNetV2-u8 graph (reduced 96x96 input) through the operator list, every layer bit-exact."""
    import importlib
    import mobilenet_ref
    mn = importlib.import_module("cl_eden_kernel_b200.mobilenet")
    layers, _ = mn.build_model(seed=3, calib_images=1, resolution=96, num_classes=100)
    x = np.random.default_rng(7).integers(0, 256, (3, 96, 96, 3), dtype=np.int64).astype(np.uint8)
    y_ref, acts = mobilenet_ref.run_oracle(layers, x, keep=True)
    ol, info = mn.make_oplist(enn, ctx, layers, batch=3, resolution=96)
    try:
        (y,) = ol.execute([x])
        # intermediate tensors share pooled buffers, so compare the ones still live plus the output
        assert np.array_equal(y.reshape(y_ref.shape), y_ref)
        (y2,) = ol.execute([x])                      # graph replay gives the same answer
        assert np.array_equal(y, y2)
        st = ol.stats()
        assert st["buffers"] < len(layers)           # liveness-based reuse happened
        assert len(np.unique(y_ref)) > 20
    finally:
        ol.destroy()


def test_oplist_with_deconvolution(enn, orc, ctx):
    """conv -> transposed conv -> conv in one operator list: the deconvolution's parity-class launches fork onto side
    streams inside the captured graph and join again; results equal the oracle chain, twice (graph replay)."""
    d1, x, w1, b1, s1 = cases.conv_case(seed=21, n=2, h=12, w=12, cin=16, cout=32, k=3, per_channel=True, out_scale=0.2)
    y1 = orc.conv2d(d1, x, w1, b1, s1)
    d2, _, w2, b2, s2 = cases.deconv_case(seed=22, n=2, h=12, w=12, cin=32, cout=16, in_zp=int(d1.out_zp), in_scale=float(d1.out_scale))
    y2 = orc.deconv(d2, y1, w2, b2, s2)
    oh, ow = y2.shape[1], y2.shape[2]
    d3, _, w3, b3, s3 = cases.conv_case(seed=23, n=2, h=oh, w=ow, cin=16, cout=16, k=1, per_channel=True, out_scale=0.1,
                                        in_zp=int(d2.out_zp), in_scale=float(d2.out_scale))
    y3 = orc.conv2d(d3, y2, w3, b3, s3)
    ol = enn.OpList(ctx)
    ops = [enn.conv2d(ctx, d1, w1, b1, s1), enn.deconv(ctx, d2, w2, b2, s2), enn.conv2d(ctx, d3, w3, b3, s3)]
    try:
        t0 = ol.tensor(x.nbytes)
        t1, t2, t3 = ol.tensor(y1.nbytes), ol.tensor(y2.nbytes), ol.tensor(y3.nbytes)
        ol.add(ops[0], [t0], t1)
        ol.add(ops[1], [t1], t2)
        ol.add(ops[2], [t2], t3)
        ol.set_io([t0], [t3], [y3.nbytes])
        ol.finalize()
        for _ in range(2):
            (y,) = ol.execute([x])
            assert np.array_equal(y.reshape(y3.shape), y3)
    finally:
        ol.destroy()


@pytest.mark.parametrize("out_stream", [True, False])
def test_oplist_pipelined_submit(enn, out_stream):
    """enn_b200_oplist_submit / wait (copy-in overlapped with the previous graph, results on their own stream or, with
    option no_out_stream, on the operators' stream) gives the blocking call's results."""
    import importlib
    mn = importlib.import_module("cl_eden_kernel_b200.mobilenet")
    layers, _ = mn.build_model(seed=4, calib_images=1, resolution=64, num_classes=50)
    ctx = enn.Context(0)
    if not out_stream:
        ctx.set_option("no_out_stream", 1)
    ol, info = mn.make_oplist(enn, ctx, layers, batch=2, resolution=64)
    try:
        rng = np.random.default_rng(11)
        xs = [rng.integers(0, 256, (2, 64, 64, 3), dtype=np.int64).astype(np.uint8) for _ in range(5)]
        want = [ol.execute([x])[0].copy() for x in xs]
        outs = [np.zeros(100, np.uint8) for _ in xs]
        for x, o in zip(xs, outs):
            ol.submit_host_ptrs([x.ctypes.data], [o.ctypes.data])
        ol.wait()
        for w, o in zip(want, outs):
            assert np.array_equal(w, o)
        assert len({w.tobytes() for w in want}) == len(want)      # the five inputs really gave five different results
    finally:
        ol.destroy()
        ctx.close()


def test_oplist_submit_round_and_sm_share(enn, orc):
    """Three operator lists in their own contexts, each limited to a share of the SMs (option grid_cap), fed in rounds
    (enn_b200_oplist_submit_round: all inputs first, then the graphs together): every result equals the oracle, the
    same lists through plain submit give the same bytes, and a bad round is refused."""
    import importlib
    import mobilenet_ref
    mn = importlib.import_module("cl_eden_kernel_b200.mobilenet")
    layers, _ = mn.build_model(seed=8, calib_images=1, resolution=64, num_classes=40)
    rng = np.random.default_rng(13)
    n_lists, rounds, batch = 3, 4, 2
    xs = [[rng.integers(0, 256, (batch, 64, 64, 3), dtype=np.int64).astype(np.uint8) for _ in range(n_lists)] for _ in range(rounds)]
    want = [[mobilenet_ref.run_oracle(layers, x).reshape(-1) for x in row] for row in xs]
    ctxs = [enn.Context(0) for _ in range(n_lists)]
    for c in ctxs:
        c.set_option("grid_cap", 5)
    lists = [mn.make_oplist(enn, c, layers, batch=batch, resolution=64)[0] for c in ctxs]
    try:
        outs = [[np.zeros(batch * 40, np.uint8) for _ in range(n_lists)] for _ in range(rounds)]
        for r in range(rounds):
            k = n_lists if r != 2 else 2                # one round with fewer lists than the others
            enn.OpList.submit_round(lists[:k], [[x.ctypes.data] for x in xs[r][:k]], [[o.ctypes.data] for o in outs[r][:k]])
            for l, x, o in zip(lists[k:], xs[r][k:], outs[r][k:]):
                l.submit_host_ptrs([x.ctypes.data], [o.ctypes.data])
        for l in lists:
            l.wait()
        for r in range(rounds):
            for o, w in zip(outs[r], want[r]):
                assert np.array_equal(o, w)
        # refusals: the same list twice, an empty round
        import ctypes as C
        hs = (C.c_void_p * 2)(lists[0].h, lists[0].h)
        buf = (C.c_void_p * 1)(xs[0][0].ctypes.data)
        tab = (C.POINTER(C.c_void_p) * 2)(C.cast(buf, C.POINTER(C.c_void_p)), C.cast(buf, C.POINTER(C.c_void_p)))
        assert enn.lib.enn_b200_oplist_submit_round(hs, 2, tab, tab) == enn.INVALID_PARAMS
        assert enn.lib.enn_b200_oplist_submit_round(hs, 0, tab, tab) == enn.INVALID_PARAMS
    finally:
        for l in lists:
            l.destroy()
        for c in ctxs:
            c.close()


GRID_CAP_CASES = {
    "conv1x1_pack": lambda: ("conv", cases.conv_case(seed=61, n=4, h=28, w=28, cin=32, cout=192, k=1, per_channel=True, act=cases.enn.ACT_RELU6)),
    "conv3x3_tapbox": lambda: ("conv", cases.conv_case(seed=62, n=3, h=20, w=20, cin=64, cout=64, k=3, per_channel=True)),
    "conv1x1_wide_n": lambda: ("conv", cases.conv_case(seed=63, n=2, h=14, w=14, cin=96, cout=576, k=1, per_channel=True)),
    "dw_s1": lambda: ("dw", cases.depthwise_case(seed=64, n=3, h=28, w=28, c=96, stride=1)),
    "dw_s2": lambda: ("dw", cases.depthwise_case(seed=65, n=3, h=28, w=28, c=64, stride=2)),
    "deconv": lambda: ("deconv", cases.deconv_case(seed=66, n=2, h=12, w=12, cin=32, cout=16)),
}


@pytest.mark.parametrize("name", sorted(GRID_CAP_CASES))
@pytest.mark.parametrize("cap", [1, 7])
def test_grid_cap_keeps_results(enn, orc, name, cap):
    """Option grid_cap (at most that many CTAs per persistent kernel): bit-exact with the oracle whatever the share."""
    kind, (d, x, w, b, s) = GRID_CAP_CASES[name]()
    c = enn.Context(0)
    try:
        c.set_option("grid_cap", cap)
        if kind == "conv":
            op, ref = enn.conv2d(c, d, w, b, s), orc.conv2d(d, x, w, b, s)
        elif kind == "dw":
            op, ref = enn.depthwise(c, d, w, b, s), orc.depthwise(d, x, w, b, s)
        else:
            op, ref = enn.deconv(c, d, w, b, s), orc.deconv(d, x, w, b, s)
        y = op.run(x)
        assert np.array_equal(y.reshape(ref.shape), ref)
        op.release()
    finally:
        c.close()


def test_oplist_group_splits_one_batch(enn, orc):
    """enn_b200_group_*: one host batch in, one host buffer out, over three operator lists with slices of 3 + 2 + 1
    images (their own contexts; on a one-GPU machine all on device 0): blocking and pipelined calls equal the oracle on
    the whole batch."""
    import importlib
    import mobilenet_ref
    mn = importlib.import_module("cl_eden_kernel_b200.mobilenet")
    layers, _ = mn.build_model(seed=6, calib_images=1, resolution=64, num_classes=40)
    rng = np.random.default_rng(12)
    xs = [rng.integers(0, 256, (6, 64, 64, 3), dtype=np.int64).astype(np.uint8) for _ in range(3)]
    want = [mobilenet_ref.run_oracle(layers, x).reshape(-1) for x in xs]
    ctxs = [enn.Context(0) for _ in range(3)]
    lists = [mn.make_oplist(enn, c, layers, batch=b, resolution=64)[0] for c, b in zip(ctxs, (3, 2, 1))]
    grp = enn.Group(lists)
    try:
        for x, w in zip(xs, want):
            (y,) = grp.execute([x])
            assert np.array_equal(y, w)
        outs = [np.zeros(6 * 40, np.uint8) for _ in xs]
        for x, o in zip(xs, outs):
            grp.submit_host_ptrs([x.ctypes.data], [o.ctypes.data])
        grp.wait()
        for o, w in zip(outs, want):
            assert np.array_equal(o, w)
    finally:
        grp.destroy()
        for c in ctxs:
            c.close()


def test_mobilenet_layers_individually(enn, orc, ctx):
    """Each distinct MobileNetV2 layer shape at 224x224, batch 2, fed with the oracle's own activations."""
    import importlib
    import mobilenet_ref
    mn = importlib.import_module("cl_eden_kernel_b200.mobilenet")
    layers, _ = mn.build_model(seed=1, calib_images=1)
    x = np.random.default_rng(8).integers(0, 256, (2, 224, 224, 3), dtype=np.int64).astype(np.uint8)
    _, acts = mobilenet_ref.run_oracle(layers, x, keep=True)
    for L in layers:
        d = mn.layer_descs(enn, L, 2)
        a = acts[L["src"]]
        if L["kind"] == "conv":
            op = enn.conv2d(ctx, d, L["w"], L["bias"], L["scales"])
        elif L["kind"] == "dw":
            op = enn.depthwise(ctx, d, L["w"], L["bias"], L["scales"])
        elif L["kind"] == "fc":
            op = enn.fully_connected(ctx, d, L["w"].reshape(L["cout"], L["cin"]), L["bias"], L["scales"])
        elif L["kind"] == "add":
            op = enn.add(ctx, d)
        else:
            op = enn.avgpool(ctx, d)
        try:
            y = op.run(a, acts[L["src2"]] if L["kind"] == "add" else None)
            assert np.array_equal(y, acts[L["name"]].reshape(-1)), L["name"]
        finally:
            op.release()


def test_cpp_adapter_interface(enn):
    """Builds and runs tests/adapter_test.cpp: the reference KAT and seeded operators through the C++ classes that
    mirror the CL* operators (initialize / execute / release on ITensor inputs)."""
    import subprocess
    root = os.path.dirname(HERE)
    pkg = os.path.join(root, "cl-eden-kernel_b200")
    exe = os.path.join(root, "tests", "adapter_test.bin")
    subprocess.run(["make", "-C", pkg, "libenn_b200_adapter.so"], check=True, capture_output=True)
    subprocess.run(["make", "-C", os.path.join(root, "oracle"), "liboracle.so"], check=True, capture_output=True)
    subprocess.run(["/usr/bin/g++", "-O1", "-std=c++17", "-o", exe, os.path.join(HERE, "adapter_test.cpp"),
                    "-L" + pkg, "-lenn_b200_adapter", "-lenn_b200", "-L" + os.path.join(root, "oracle"), "-loracle",
                    "-Wl,-rpath," + pkg, "-Wl,-rpath," + os.path.join(root, "oracle"), "-fopenmp"], check=True, capture_output=True)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "adapter test: OK" in r.stdout, r.stdout + r.stderr
    # The same program built against the reference's own ITensor / Common / parameter headers (tests/test_adapter_cpu.py
    # builds it where the reference tree is mounted); it is run when it is there.
    ref_exe = os.path.join(HERE, "adapter_test_refhdr.bin")
    if os.path.exists(ref_exe):
        r = subprocess.run([ref_exe], capture_output=True, text=True, timeout=120)
        assert r.returncode == 0 and "adapter test: OK" in r.stdout, r.stdout + r.stderr


@pytest.mark.parametrize("name", list(__import__("ref_cases").CASES))
def test_library_matches_reference_kernel_text_golden(enn, ctx, name):
    """The CUDA path through the C ABI against outputs of the reference's own kernel text (tests/golden/ref_kernels.npz)."""
    import ref_cases
    golden = np.load(os.path.join(HERE, "golden", "ref_kernels.npz"))[name]
    kind, mk = ref_cases.CASES[name]
    case = mk()
    if kind in ("maxpool", "mean", "resize", "concat"):
        d, x = case
        op = {"maxpool": enn.maxpool, "mean": enn.mean, "resize": enn.resize_bilinear, "concat": enn.concat}[kind](ctx, d)
        try:
            y = op.run_n(x) if kind == "concat" else op.run(x)
            assert np.array_equal(y, golden.reshape(-1)), name
        finally:
            op.release()
        return
    if kind in ("conv_pc", "conv_pt", "dw", "deconv"):
        d, x, w, b, sc = case
        op = {"conv_pc": enn.conv2d, "conv_pt": enn.conv2d, "dw": enn.depthwise, "deconv": enn.deconv}[kind](ctx, d, w, b, sc)
        x2 = None
    elif kind == "pool":
        d, x = case
        op, x2 = enn.avgpool(ctx, d), None
    else:
        d, x, x2 = case
        op = enn.add(ctx, d)
    try:
        for impl in _impls(enn, op) if kind in ("conv_pc", "conv_pt", "deconv") else [op.info.impl]:
            op.set_impl(impl)
            assert np.array_equal(op.run(x, x2), golden.reshape(-1)), (name, impl)
    finally:
        op.release()


# ---- remaining graph operators (MaxPool, Mean, Concat, Softmax, Resize) against the oracle ----
@pytest.mark.parametrize("shape", [(2, 9, 11, 6, 3, 2, 1, "u8", 0), (1, 112, 112, 24, 3, 2, 0, "u8", 3), (3, 7, 7, 40, 2, 1, 0, "s8", 0),
                                   (1, 5, 6, 3, 5, 1, 2, "s8", 1)])
def test_maxpool_parity(enn, orc, ctx, shape):
    n, h, w, c, k, s, pad, dt, act = shape
    signed = dt == "s8"
    x = np.random.default_rng(h * w + c).integers(-128 if signed else 0, 128 if signed else 256, (n, h, w, c), dtype=np.int64).astype(np.int8 if signed else np.uint8)
    oh, ow = (h - k + s + 2 * pad) // s, (w - k + s + 2 * pad) // s
    d = enn.PoolDesc(n=n, h=h, w=w, c=c, kh=k, kw=k, stride_h=s, stride_w=s, pad_t=pad, pad_l=pad, out_h=oh, out_w=ow, activation=act,
                     act_dtype=enn.S8 if signed else enn.U8, out_scale=0.04, out_zp=-20 if signed else 7)
    op = enn.maxpool(ctx, d)
    try:
        _check(op, orc.maxpool(d, x), x)
    finally:
        op.release()


@pytest.mark.parametrize("dims,axes,dt", [((4, 7, 7, 1280), (1, 2), "u8"), ((2, 9, 5, 33), (3,), "u8"), ((3, 4, 6, 8), (0, 2), "s8"),
                                          ((2, 3, 5, 7), (0, 1, 2, 3), "s8"), ((1, 1, 40, 17), (2,), "u8")])
def test_mean_parity(enn, orc, ctx, dims, axes, dt):
    signed = dt == "s8"
    x = np.random.default_rng(sum(dims)).integers(-128 if signed else 0, 128 if signed else 256, dims, dtype=np.int64).astype(np.int8 if signed else np.uint8)
    d = enn.mean_desc(dims, axes, enn.S8 if signed else enn.U8)
    op = enn.mean(ctx, d)
    try:
        _check(op, orc.mean(d, x), x)
    finally:
        op.release()


@pytest.mark.parametrize("outer,inner,dt", [(56 * 56 * 2, (24, 24, 48), "u8"), (3, (1000, 7), "u8"), (17, (5, 3, 9, 2, 8, 1, 4, 6), "s8"), (1, (33,), "u8")])
def test_concat_parity(enn, orc, ctx, outer, inner, dt):
    signed = dt == "s8"
    rng = np.random.default_rng(outer + len(inner))
    xs = [rng.integers(-128 if signed else 0, 128 if signed else 256, (outer, k), dtype=np.int64).astype(np.int8 if signed else np.uint8) for k in inner]
    scales = [0.02 if i % 3 == 0 else float(rng.uniform(0.005, 0.08)) for i in range(len(inner))]      # every third input: plain copy
    zps = [int(rng.integers(-20, 20) if signed else rng.integers(0, 256)) for _ in inner]
    d = enn.concat_desc(outer, inner, scales, zps, 0.02, -3 if signed else 120, enn.S8 if signed else enn.U8)
    op = enn.concat(ctx, d)
    try:
        y = op.run_n(xs).reshape(outer, sum(inner))
        assert np.array_equal(y, orc.concat(d, xs))
    finally:
        op.release()


@pytest.mark.parametrize("outer,channels,inner,beta,dt", [(256, 1000, 1, 1.0, "u8"), (2, 21, 65, 1.0, "u8"), (7, 10, 1, 0.5, "s8"), (1, 1, 9, 2.0, "u8")])
def test_softmax_parity(enn, orc, ctx, outer, channels, inner, beta, dt):
    """Quantized softmax = dequantise, float softmax, quantise.  The library and the oracle take exp() from the same host
    libm and keep every float operation separate, so the bytes are equal; against the reference's OpenCL exp() a last-
    bit difference of the exponential can move an output by one step."""
    signed = dt == "s8"
    x = np.random.default_rng(channels).integers(-128 if signed else 0, 128 if signed else 256, (outer, channels, inner), dtype=np.int64).astype(np.int8 if signed else np.uint8)
    d = enn.SoftmaxDesc(outer=outer, channels=channels, inner=inner, beta=beta, act_dtype=enn.S8 if signed else enn.U8, in_scale=0.05,
                        in_zp=-3 if signed else 121, out_scale=1.0 / 256, out_zp=-128 if signed else 0)
    op = enn.softmax(ctx, d)
    try:
        y = op.run(x).reshape(x.shape)
        y_ref = orc.softmax(d, x)
        assert np.array_equal(y, y_ref)
        assert len(np.unique(y_ref)) > (3 if channels > 1 else 0)
    finally:
        op.release()


@pytest.mark.parametrize("shape", [(2, 5, 6, 4, 10, 13, 0, 0, "u8"), (1, 33, 33, 21, 129, 129, 1, 0, "u8"), (2, 9, 8, 16, 4, 5, 0, 1, "s8"),
                                   (1, 1, 1, 8, 7, 3, 1, 0, "u8"), (1, 16, 16, 32, 32, 32, 0, 1, "u8")])
def test_resize_bilinear_parity(enn, orc, ctx, shape):
    n, h, w, c, oh, ow, align, half, dt = shape
    signed = dt == "s8"
    x = np.random.default_rng(h * ow).integers(-128 if signed else 0, 128 if signed else 256, (n, h, w, c), dtype=np.int64).astype(np.int8 if signed else np.uint8)
    d = enn.ResizeDesc(n=n, h=h, w=w, c=c, out_h=oh, out_w=ow, align_corners=align, half_pixel_centers=half, act_dtype=enn.S8 if signed else enn.U8)
    op = enn.resize_bilinear(ctx, d)
    try:
        _check(op, orc.resize_bilinear(d, x), x)
    finally:
        op.release()


def test_oplist_with_graph_operators(enn, orc, ctx):
    """conv -> {maxpool, resize} -> concat -> mean -> softmax in one operator list (a concatenation node with two inputs)."""
    d1, x, w1, b1, s1 = cases.conv_case(seed=31, n=2, h=16, w=16, cin=8, cout=16, k=3, per_channel=True, out_scale=0.2)
    y1 = orc.conv2d(d1, x, w1, b1, s1)
    dp = enn.PoolDesc(n=2, h=16, w=16, c=16, kh=2, kw=2, stride_h=2, stride_w=2, pad_t=0, pad_l=0, out_h=8, out_w=8, activation=0, act_dtype=enn.U8,
                      out_scale=float(d1.out_scale), out_zp=int(d1.out_zp))
    y2 = orc.maxpool(dp, y1)
    dr = enn.ResizeDesc(n=2, h=16, w=16, c=16, out_h=8, out_w=8, align_corners=0, half_pixel_centers=1, act_dtype=enn.U8)
    y3 = orc.resize_bilinear(dr, y1)
    dc = enn.concat_desc(2 * 8 * 8, (16, 16), (float(d1.out_scale), float(d1.out_scale)), (int(d1.out_zp), int(d1.out_zp)), 0.3, 100)
    y4 = orc.concat(dc, [y2.reshape(-1, 16), y3.reshape(-1, 16)])
    dm = enn.mean_desc((2, 8, 8, 32), (1, 2))
    y5 = orc.mean(dm, y4.reshape(2, 8, 8, 32))
    ds = enn.SoftmaxDesc(outer=2, channels=32, inner=1, beta=1.0, act_dtype=enn.U8, in_scale=0.3, in_zp=100, out_scale=1.0 / 256, out_zp=0)
    y6 = orc.softmax(ds, y5.reshape(2, 32, 1))
    ol = enn.OpList(ctx)
    try:
        t = [ol.tensor(v.size) for v in (x, y1, y2, y3, y4, y5, y6)]
        ol.add(enn.conv2d(ctx, d1, w1, b1, s1), [t[0]], t[1])
        ol.add(enn.maxpool(ctx, dp), [t[1]], t[2])
        ol.add(enn.resize_bilinear(ctx, dr), [t[1]], t[3])
        ol.add(enn.concat(ctx, dc), [t[2], t[3]], t[4])
        ol.add(enn.mean(ctx, dm), [t[4]], t[5])
        ol.add(enn.softmax(ctx, ds), [t[5]], t[6])
        ol.set_io([t[0]], [t[6]], [y6.size])
        ol.finalize()
        for _ in range(2):
            (y,) = ol.execute([x])
            assert np.array_equal(y, y6.reshape(-1))
    finally:
        ol.destroy()
