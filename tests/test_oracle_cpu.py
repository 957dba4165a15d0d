"""CPU tests: the oracle against the reference's golden material, and the library's host-side helpers."""
import ctypes as C
import json
import os
import re

import numpy as np
import pytest

import cases

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


@pytest.fixture(scope="module")
def golden():
    with open(os.path.join(HERE, "golden", "quant_host.json")) as f:
        return json.load(f)


def test_quantize_multiplier_golden(orc, enn, golden):
    for m, qm, sh in golden["quantize_multiplier"]:
        assert orc.quantize_multiplier(m) == (qm, sh)
        a, b = C.c_int32(), C.c_int32()
        enn.lib.enn_b200_quantize_multiplier(m, C.byref(a), C.byref(b))
        assert (a.value, b.value) == (qm, sh)


def test_conv_multiplier_golden(orc, enn, golden):
    for a, b, bs, o, st, m in golden["conv_multiplier"]:
        st2, m2 = orc.conv_multiplier(a, b, bs, o)
        assert (st2, m2) == (st, m)
        mm = C.c_double(0.0)
        st3 = enn.lib.enn_b200_conv_multiplier(a, b, bs, o, C.byref(mm))
        assert (st3, mm.value) == (st, m)


def test_activation_range_golden(orc, enn, golden):
    for act, dt, scale, zp, lo, hi in golden["activation_range"]:
        assert orc.activation_range(act, dt, scale, zp) == (lo, hi)
        a, b = C.c_int32(), C.c_int32()
        enn.lib.enn_b200_activation_range(act, dt, scale, zp, C.byref(a), C.byref(b))
        assert (a.value, b.value) == (lo, hi)


def test_fixed_point_golden(orc, enn, golden):
    for a, b, r in golden["srdhm"]:
        assert orc.lib.orc_srdhm(a, b) == r
    for x, e, r in golden["rdivpot"]:
        assert orc.lib.orc_rdivpot(x, e) == r
    for x, qm, sh, r in golden["multiply_by_quantized_multiplier"]:
        # zero point 0 and the widest clamp turn the kernel tail into MultiplyByQuantizedMultiplier
        assert orc.lib.orc_requant(x, qm, sh, 0, -2**31, 2**31 - 1) == r
        assert enn.lib.enn_b200_requant_host(x, qm, sh, 0, -2**31, 2**31 - 1) == r


def test_oracle_matches_reference_build(orc):
    """Where the reference tree was available at build time, compare with its own code on fresh inputs."""
    if orc.ref is None:
        pytest.skip("oracle/_ref not built (reference tree absent)")
    rng = np.random.default_rng(1)
    for _ in range(2000):
        m = float(np.exp(rng.uniform(np.log(1e-8), np.log(64.0))))
        assert orc.quantize_multiplier(m) == orc.quantize_multiplier(m, orc.ref)
        a = int(rng.integers(-2**31, 2**31))
        b = int(rng.integers(2**30, 2**31))
        assert orc.lib.orc_srdhm(a, b) == orc.ref.ref_srdhm(a, b)
        e = int(rng.integers(0, 32))
        assert orc.lib.orc_rdivpot(a, e) == orc.ref.ref_rdivpot(a, e)
        act, dt = int(rng.integers(0, 4)), int(rng.integers(0, 2))
        sc = float(np.float32(np.exp(rng.uniform(np.log(1e-3), 0.0))))
        zp = int(rng.integers(-128, 128)) if dt else int(rng.integers(0, 256))
        assert orc.activation_range(act, dt, sc, zp) == orc.activation_range(act, dt, sc, zp, orc.ref)


def test_device_requant_formula_exhaustive_ties(orc, enn):
    """The single-shift form of stage 1 used on the device equals the reference's nudge/truncate form."""
    rng = np.random.default_rng(2)
    mults = [2**30, 2**30 + 1, 2**31 - 1, 1518500250] + [int(v) for v in rng.integers(2**30, 2**31, 40)]
    accs = list(range(-300, 301)) + [int(v) for v in rng.integers(-2**31, 2**31, 300)]
    for m in mults:
        for sh in (-12, -8, -3, -1, 0):
            for a in accs:
                assert enn.lib.enn_b200_requant_host(a, m, sh, 7, -2**31, 2**31 - 1) == \
                    orc.lib.orc_requant(a, m, sh, 7, -2**31, 2**31 - 1)
    assert enn.lib.enn_b200_requant_host(-2**31, -2**31, 0, 0, -2**31, 2**31 - 1) == 2**31 - 1


def _kat():
    with open(os.path.join(HERE, "golden", "kat_perchannel_conv.json")) as f:
        return json.load(f)


def test_kat_perchannel_conv_oracle(orc, enn):
    """Reference known-answer test gpu_userdriver_test.cc:474-575 (includes the exact -6.5 -> -7 tie)."""
    k = _kat()
    n, c, h, w = k["input_dims_nchw"]
    x = np.array(k["input"], np.uint8).reshape(n, c, h, w).transpose(0, 2, 3, 1)      # NCHW -> NHWC
    wt = np.array(k["weight"], np.int8).reshape(k["weight_dims_ohwi"])
    d = enn.conv_desc(n=n, h=h, w=w, cin=c, cout=3, kh=1, kw=1, per_channel=1, weight_dtype=enn.S8,
                      weight_layout=enn.W_OHWI, in_scale=k["input_scale"], in_zp=k["zero_point"],
                      out_scale=k["output_scale"], out_zp=k["zero_point"])
    y = orc.conv2d(d, x, wt, np.array(k["bias"], np.int32), np.array(k["scales"], np.float32))
    assert y.transpose(0, 3, 1, 2).reshape(-1).tolist() == k["expect"]


def test_oracle_conv_against_numpy_float_model(orc, enn):
    """Independent check of index order: small integers, unit scales, so the float convolution is exact."""
    rng = np.random.default_rng(3)
    for layout in (enn.W_OHWI, enn.W_OIHW):
        d, x, wt, bias, _ = cases.conv_case(seed=5, n=2, h=7, w=6, cin=4, cout=6, k=3, stride=2, groups=2,
                                            layout=layout, act=enn.ACT_NONE, in_scale=1.0, in_zp=3, w_scale=1.0,
                                            w_zp=2, out_scale=1.0, out_zp=100, bias_range=5)
        x = (x % 7).astype(np.uint8)
        wt = (wt % 5).astype(np.uint8)
        y = orc.conv2d(d, x, wt, bias)
        w_ohwi = wt if layout == enn.W_OHWI else wt.transpose(0, 2, 3, 1)
        oh, ow = y.shape[1:3]
        ref = np.zeros(y.shape, np.int64)
        xp = np.full((2, 7 + d.pad_t + d.pad_b, 6 + d.pad_l + d.pad_r, 4), 3, np.int64)
        xp[:, d.pad_t:d.pad_t + 7, d.pad_l:d.pad_l + 6] = x
        for oc in range(6):
            g = oc // 3
            for oy in range(oh):
                for ox in range(ow):
                    patch = xp[:, oy * 2:oy * 2 + 3, ox * 2:ox * 2 + 3, g * 2:g * 2 + 2] - 3
                    ref[:, oy, ox, oc] = (patch * (w_ohwi[oc].astype(np.int64) - 2)).sum(axis=(1, 2, 3)) + bias[oc]
        assert np.array_equal(np.clip(ref + 100, 0, 255).astype(np.uint8), y)


def test_oracle_deconv_against_scatter_model(orc, enn):
    """Transposed conv written the other way round (scatter from each input pixel) gives the same numbers."""
    d, x, wt, bias, _ = cases.deconv_case(seed=7, n=1, h=5, w=4, cin=3, cout=2, k=4, stride=2, pad=1,
                                          in_scale=1.0, in_zp=1, w_scale=1.0, w_zp=2, out_scale=1.0, out_zp=90)
    x = (x % 5).astype(np.uint8)
    wt = (wt % 6).astype(np.uint8)
    y = orc.deconv(d, x, wt, bias)
    oh, ow = y.shape[1:3]
    assert (oh, ow) == (10, 8)
    acc = np.zeros((1, oh + 2, ow + 2, 2), np.int64)
    for iy in range(5):
        for ix in range(4):
            for ky in range(4):
                for kx in range(4):
                    for co in range(2):
                        acc[0, iy * 2 + ky, ix * 2 + kx, co] += ((x[0, iy, ix].astype(np.int64) - 1) *
                                                                 (wt[:, co, ky, kx].astype(np.int64) - 2)).sum()
    ref = acc[:, 1:1 + oh, 1:1 + ow] + bias
    assert np.array_equal(np.clip(ref + 90, 0, 255).astype(np.uint8), y)


def test_oracle_depthwise_and_fc_small(orc, enn):
    d, x, wt, bias, sc = cases.depthwise_case(seed=9, n=1, h=5, w=5, c=4, dm=2, stride=2)
    y = orc.depthwise(d, x, wt, bias, sc)
    assert y.shape == (1, 3, 3, 8)
    # depthwise with multiplier dm equals a grouped conv with groups = C, cout/g = dm
    dc = enn.conv_desc(**{f: getattr(d, f) for f, _ in d._fields_})
    dc.groups = 4
    assert np.array_equal(orc.conv2d(dc, x, wt.reshape(8, 1, 3, 3), bias, sc), y)
    fd, fx, fw, fb, fs = cases.fc_case(seed=11, m=3, k=40, n=5)
    fy = orc.fully_connected(fd, fx, fw, fb, fs)
    cd = enn.conv_desc(n=3, h=1, w=1, cin=40, cout=5, kh=1, kw=1, per_channel=1, weight_dtype=enn.S8,
                       in_scale=fd.in_scale, in_zp=fd.in_zp, out_scale=fd.out_scale, out_zp=fd.out_zp)
    assert np.array_equal(orc.conv2d(cd, fx.reshape(3, 1, 1, 40), fw.reshape(5, 1, 1, 40), fb, fs).reshape(3, 5), fy)


def test_bias_scale_mismatch_yields_zero_point(orc, enn):
    """KernelUtil.cpp:14-16: a bias scale that is not in*w leaves the multiplier 0, so every output is out_zp."""
    d, x, wt, bias, _ = cases.conv_case(seed=1, h=6, w=6, cin=4, cout=4, act=enn.ACT_NONE)
    d.bias_scale = 0.5
    assert np.all(orc.conv2d(d, x, wt, bias) == d.out_zp)


def test_abi_exports_every_declared_symbol(enn):
    header = open(os.path.join(ROOT, "include", "enn_b200.h")).read()
    declared = set(re.findall(r"\b(enn_b200_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(enn.PROTOTYPES), declared ^ set(enn.PROTOTYPES)
    for name in declared:
        assert hasattr(enn.lib, name), name


def test_struct_sizes_match_header(enn):
    assert C.sizeof(enn.ConvDesc) == 32 * 4
    assert C.sizeof(enn.FcDesc) == 16 * 4
    assert C.sizeof(enn.AddDesc) == 8 + 8 * 4
    assert C.sizeof(enn.PoolDesc) == 16 * 4


# ---------------------------------------------------------------------------------------------------------
# Outputs of the reference's own OpenCL C kernel text (compiled as C++ and run on the CPU when the reference tree
# was mounted; tests/golden/gen_ref_kernels.py) pin the oracle's kernel restatements.
# ---------------------------------------------------------------------------------------------------------
import ref_cases  # noqa: E402


@pytest.fixture(scope="module")
def ref_golden():
    return np.load(os.path.join(HERE, "golden", "ref_kernels.npz"))


@pytest.mark.parametrize("name", list(ref_cases.CASES))
def test_oracle_matches_reference_kernel_text_golden(orc, ref_golden, name):
    kind, mk = ref_cases.CASES[name]
    got = ref_cases.run_oracle(orc, kind, mk())
    assert np.array_equal(got, ref_golden[name]), name


def test_oracle_softmax_against_float64_model(orc, enn):
    """Softmax has no integer definition; the oracle's float path stays within one output step of a float64 model."""
    rng = np.random.default_rng(5)
    x = rng.integers(0, 256, (6, 37, 3), dtype=np.int64).astype(np.uint8)
    d = enn.SoftmaxDesc(outer=6, channels=37, inner=3, beta=1.0, act_dtype=enn.U8, in_scale=0.04, in_zp=100, out_scale=1.0 / 256, out_zp=0)
    y = orc.softmax(d, x).astype(np.int64)
    real = (x.astype(np.float64) - 100) * np.float64(np.float32(0.04))
    e = np.exp(real - real.max(axis=1, keepdims=True))
    model = np.clip(np.round(e / e.sum(axis=1, keepdims=True) * 256), 0, 255)
    assert np.abs(y - model).max() <= 1 and (y != model).mean() < 0.02


def test_oracle_matches_reference_kernel_text_live(orc):
    """Fresh random geometry against the live build of the reference kernels (this container only)."""
    if not orc.has_ref_kernels():
        pytest.skip("oracle/_ref kernel shim not built (reference tree absent)")
    rng = np.random.default_rng(77)
    for i in range(12):
        h, w = int(rng.integers(3, 12)), int(rng.integers(3, 12))
        stride = int(rng.integers(1, 3))
        c = cases.conv_case(seed=200 + i, n=int(rng.integers(1, 3)), h=h, w=w, cin=int(rng.integers(1, 9)), cout=int(rng.integers(1, 9)),
                            k=int(rng.choice([1, 3])), stride=stride, per_channel=True, out_scale=float(rng.uniform(0.05, 0.5)),
                            out_zp=int(rng.integers(0, 256)), act=int(rng.integers(0, 4)))
        assert np.array_equal(orc.conv2d(*c), orc.ref_conv_per_channel(*c))
        groups = int(rng.choice([1, 1, 2]))
        t = cases.conv_case(seed=250 + i, n=int(rng.integers(1, 3)), h=h + 1, w=w + 1, cin=groups * int(rng.integers(1, 7)),
                            cout=groups * int(rng.integers(1, 10)), kh=int(rng.choice([1, 3, 5])), kw=int(rng.choice([1, 3, 5, 7])), stride=stride,
                            groups=groups, layout=int(rng.choice([cases.enn.W_OIHW, cases.enn.W_OHWI])), w_zp=int(rng.integers(0, 256)),
                            in_zp=int(rng.integers(0, 256)), out_scale=float(rng.uniform(0.02, 0.3)), out_zp=int(rng.integers(0, 256)),
                            act=int(rng.integers(0, 4)), pad=str(rng.choice(["same", "valid"])) if h > 6 and w > 8 else "same")
        assert np.array_equal(orc.conv2d(*t), orc.ref_conv_per_tensor(*t[:4]))
        for pc in (True, False):
            dcase = cases.depthwise_case(seed=300 + i, n=1, h=h + 2, w=w + 2, c=int(rng.integers(1, 7)), stride=stride, per_channel=pc,
                                         out_scale=float(rng.uniform(0.02, 0.2)), out_zp=int(rng.integers(0, 200)), act=int(rng.integers(0, 4)),
                                         dm=int(rng.integers(1, 3)))
            assert np.array_equal(orc.depthwise(*dcase), orc.ref_depthwise(*dcase))
            k = int(rng.choice([2, 3, 4]))
            tcase = cases.deconv_case(seed=400 + i, n=1, h=min(h, 6), w=min(w, 6), cin=int(rng.integers(1, 10)), cout=int(rng.integers(1, 6)), k=k,
                                      stride=int(rng.integers(1, 3)), pad=int(rng.integers(0, 2)), per_channel=pc,
                                      layout=int(rng.choice([cases.enn.W_IOHW, cases.enn.W_OHWI])), out_scale=float(rng.uniform(0.05, 0.6)))
            assert np.array_equal(orc.deconv(*tcase), orc.ref_deconv(*tcase))
        # remaining graph operators against the reference's maxpooling, mean_feature_opt / sum_axis / mean, concat_axis1, resize_bilinear
        import ref_cases
        k, st = int(rng.integers(1, 4)), int(rng.integers(1, 3))
        mp = ref_cases._maxpool(500 + i, 1, h + 2, w + 3, int(rng.integers(1, 6)), k, st, int(rng.integers(0, k)), act=int(rng.integers(0, 4)))
        assert np.array_equal(orc.maxpool(*mp), orc.ref_maxpool(*mp))
        dims = tuple(int(v) for v in rng.integers(1, 8, 4))
        axes = tuple(a for a in range(4) if rng.integers(0, 2)) or (3,)
        mc = ref_cases._mean(600 + i, dims, axes)
        assert np.array_equal(orc.mean(*mc), orc.ref_mean(*mc)), (dims, axes)
        inner = tuple(int(v) for v in rng.integers(1, 9, int(rng.integers(1, 5))))
        cc = ref_cases._concat(700 + i, int(rng.integers(1, 20)), inner, [float(rng.choice([0.02, rng.uniform(0.004, 0.09)])) for _ in inner],
                               [int(v) for v in rng.integers(0, 256, len(inner))], 0.02, int(rng.integers(0, 256)))
        assert np.array_equal(ref_cases.run_oracle(orc, "concat", cc), ref_cases.run_reference(orc, "concat", cc))
        rc = ref_cases._resize(800 + i, 1, h, w, int(rng.integers(1, 5)), int(rng.integers(1, 20)), int(rng.integers(1, 20)), align=int(rng.integers(0, 2)),
                               half=int(rng.integers(0, 2)))
        assert np.array_equal(orc.resize_bilinear(*rc), orc.ref_resize_bilinear(*rc))
