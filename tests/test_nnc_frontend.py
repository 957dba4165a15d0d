"""NNC (v2) front end: model files written by tests/nnc_writer.py are (a) checked with the reference's own generated
flatbuffer reader and verifier where the reference tree is mounted (CPU), and (b) loaded through enn_b200_model_open and
compared with the operator lists built call by call and with the oracle (GPU)."""
import importlib
import os
import subprocess

import numpy as np
import pytest

import cases
import nnc_writer as nw

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
REF_SRC = "/root/reference/src"
enn = cases.enn
mn = importlib.import_module("cl_eden_kernel_b200.mobilenet")


def _small_model(resolution=32, classes=10, seed=3):
    layers, _ = mn.build_model(seed=seed, calib_images=1, resolution=resolution, num_classes=classes)
    return layers


def test_writer_output_is_valid_for_the_reference_reader(tmp_path):
    """The reference's flatbuffers verifier accepts the file and its generated accessors return what was written."""
    if not os.path.isdir(REF_SRC):
        pytest.skip("reference tree absent")
    exe = os.path.join(ROOT, "oracle", "_ref", "nnc_ref_check")
    os.makedirs(os.path.dirname(exe), exist_ok=True)
    subprocess.run(["/usr/bin/g++", "-O1", "-std=c++17", "-w", "-I" + REF_SRC, "-o", exe, os.path.join(HERE, "nnc_ref_check.cpp")], check=True)
    layers = _small_model()
    path = tmp_path / "m.nnc"
    path.write_bytes(nw.mobilenet_to_nnc(layers, 2, 32))
    r = subprocess.run([exe, str(path)], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout
    lines = r.stdout.splitlines()
    assert lines[0].startswith("model version 201 legacy 5 subgraphs 1")
    ops = [ln for ln in lines if ln.startswith("op ")]
    want_codes = {"conv": 3, "dw": 4, "fc": 9, "add": 0, "pool": 1}
    assert [int(ln.split()[3]) for ln in ops] == [want_codes[L["kind"]] for L in layers]
    first = layers[0]
    assert "shape 32 3 3 3" in lines[2] and f"pc 32 first {first['scales'][0]:.9g}" in lines[2] and "bytes 864" in lines[2]
    assert f"scale {first['in_scale']:.9g} zp 128" in lines[1]
    assert "conv pad 0 sw 2 sh 2 act 3" in ops[0]          # stem: SAME, stride 2, RELU6
    assert lines[-1] == f"inputs 0 outputs {len([ln for ln in lines if ln.startswith('tensor ')]) - 1}"


@pytest.mark.gpu
def test_nnc_mobilenet_equals_the_call_by_call_list(orc, ctx):
    import mobilenet_ref
    layers = _small_model(resolution=64, classes=50, seed=4)
    x = np.random.default_rng(21).integers(0, 256, (3, 64, 64, 3), dtype=np.int64).astype(np.uint8)
    y_ref = mobilenet_ref.run_oracle(layers, x).reshape(-1)
    model = enn.Model(ctx, nw.mobilenet_to_nnc(layers, 1, 64), batch=3)      # the file says batch 1; the caller asks for 3
    ol, _ = mn.make_oplist(enn, ctx, layers, batch=3, resolution=64)
    try:
        assert (model.n_inputs, model.n_outputs, model.n_operators) == (1, 1, len(layers))
        (y,) = model.execute([x])
        (y2,) = ol.execute([x])
        assert np.array_equal(y, y2) and np.array_equal(y, y_ref)
    finally:
        model.close()
        ol.destroy()


def _graph_model(legacy):
    """conv (SAME, stride 2) -> {maxpool, resize} -> concat -> mean(H, W) -> fc -> softmax, and (ANDROID_NN only) a
    transposed convolution branch from the conv output, as an NNC model plus the oracle's result."""
    from oracle import orc
    rng = np.random.default_rng(33)
    n, h, cin, c1 = 2, 15, 8, 16
    x = rng.integers(0, 256, (n, h, h, cin), dtype=np.int64).astype(np.uint8)
    w1 = rng.integers(0, 256, (c1, 3, 3, cin), dtype=np.int64).astype(np.uint8)
    b1 = rng.integers(-500, 500, c1, dtype=np.int64).astype(np.int32)
    mb = nw.ModelBuilder(legacy)
    t_in = mb.tensor((n, h, h, cin), "uint8", 0.02, 128)
    t_w1 = mb.tensor(w1.shape, "uint8", 0.005, 121, data=w1)
    t_b1 = mb.tensor((c1,), "int32", 0.02 * 0.005, 0, data=b1)
    oh = 8
    t_c1 = mb.tensor((n, oh, oh, c1), "uint8", 0.05, 120)
    mb.op("CONV_2D", [t_in, t_w1, t_b1], [t_c1], "Conv2DOptions", nw.Table(f0=("i8", nw.PAD_SAME), f1=("i32", 2), f2=("i32", 2), f3=("i8", 1)))
    # the reference's padding rule for this conv: total = (8 - 1) * 2 + 3 - 15 = 2 -> 1 / 1 for both model families
    d1 = enn.conv_desc(n=n, h=h, w=h, cin=cin, cout=c1, kh=3, kw=3, stride_h=2, stride_w=2, pad_t=1, pad_b=1, pad_l=1, pad_r=1, activation=1,
                       weight_layout=enn.W_OHWI, in_scale=0.02, in_zp=128, w_scale=0.005, w_zp=121, out_scale=0.05, out_zp=120)
    y1 = orc.conv2d(d1, x, w1, b1)
    t_mp = mb.tensor((n, 4, 4, c1), "uint8", 0.05, 120)
    mb.op("MAX_POOL_2D", [t_c1], [t_mp], "Pool2DOptions", nw.Table(f0=("i8", nw.PAD_VALID), f1=("i32", 2), f2=("i32", 2), f3=("i32", 2), f4=("i32", 2), f5=("i8", 0)))
    dp = enn.PoolDesc(n=n, h=oh, w=oh, c=c1, kh=2, kw=2, stride_h=2, stride_w=2, pad_t=0, pad_l=0, out_h=4, out_w=4, activation=0, act_dtype=enn.U8, out_scale=0.05, out_zp=120)
    y2 = orc.maxpool(dp, y1)
    t_rs = mb.tensor((n, 4, 4, c1), "uint8", 0.05, 120)
    mb.op("RESIZE_BILINEAR", [t_c1], [t_rs], "ResizeBilinearOptions", nw.Table(f2=("bool", 0), f3=("bool", 1)))
    dr = enn.ResizeDesc(n=n, h=oh, w=oh, c=c1, out_h=4, out_w=4, align_corners=0, half_pixel_centers=1, act_dtype=enn.U8)
    y3 = orc.resize_bilinear(dr, y1)
    t_cc = mb.tensor((n, 4, 4, 2 * c1), "uint8", 0.07, 110)
    mb.op("CONCATENATION", [t_mp, t_rs], [t_cc], "ConcatenationOptions", nw.Table(f0=("i32", 3), f1=("i8", 0)))
    dc = enn.concat_desc(n * 16, (c1, c1), (0.05, 0.05), (120, 120), 0.07, 110)
    y4 = orc.concat(dc, [y2.reshape(-1, c1), y3.reshape(-1, c1)]).reshape(n, 4, 4, 2 * c1)
    t_ax = mb.tensor((2,), "int32", data=np.array([1, 2], np.int32))
    t_mean = mb.tensor((n, 1, 1, 2 * c1), "uint8", 0.07, 110)
    mb.op("MEAN", [t_cc, t_ax], [t_mean], "ReducerOptions", nw.Table(f0=("bool", 1)))
    y5 = orc.mean(enn.mean_desc((n, 4, 4, 2 * c1), (1, 2)), y4)
    wf = rng.integers(-127, 128, (10, 2 * c1), dtype=np.int64).astype(np.int8)
    bf = rng.integers(-300, 300, 10, dtype=np.int64).astype(np.int32)
    t_wf = mb.tensor(wf.shape, "int8", 0.01, 0, data=wf)
    t_bf = mb.tensor((10,), "int32", 0.07 * 0.01, 0, data=bf)
    t_fc = mb.tensor((n, 10), "uint8", 0.1, 128)
    mb.op("FULLY_CONNECTED", [t_mean, t_wf, t_bf], [t_fc], "FullyConnectedOptions", nw.Table(f0=("i8", 0)))
    df = enn.FcDesc(m=n, k=2 * c1, n=10, activation=0, act_dtype=enn.U8, weight_dtype=enn.S8, per_channel=0, in_scale=0.07, in_zp=110, w_scale=0.01,
                    w_zp=0, bias_scale=float(np.float32(0.07) * np.float32(0.01)), out_scale=0.1, out_zp=128)
    y6 = orc.fully_connected(df, y5.reshape(n, -1), wf, bf)
    t_sm = mb.tensor((n, 10), "uint8", 1.0 / 256, 0)
    mb.op("SOFTMAX", [t_fc], [t_sm], "SoftmaxOptions", nw.Table(f0=("f32", 1.0), f1=("i32", 1)))
    y7 = orc.softmax(enn.SoftmaxDesc(outer=n, channels=10, inner=1, beta=1.0, act_dtype=enn.U8, in_scale=0.1, in_zp=128, out_scale=1.0 / 256, out_zp=0),
                     y6.reshape(n, 10, 1))
    mb.inputs, mb.outputs = [t_in], [t_sm]
    return mb.finish(), x, y7.reshape(-1)


@pytest.mark.gpu
@pytest.mark.parametrize("legacy", [nw.LEGACY_TENSORFLOW_NHWC, nw.LEGACY_CAFFE_NHWC])
def test_nnc_graph_operators(ctx, legacy):
    blob, x, want = _graph_model(legacy)
    model = enn.Model(ctx, blob)
    try:
        assert model.n_operators == 7
        (y,) = model.execute([x])
        assert np.array_equal(y, want)
    finally:
        model.close()


@pytest.mark.gpu
def test_nnc_padding_rules_differ_by_model_family(orc, ctx):
    """SAME padding with an odd total: TensorFlow-style models put the extra row / column at the end, Caffe-style models pad
    ceil(total / 2) on both sides (gpu_op_constructor.cc:1989-2005)."""
    rng = np.random.default_rng(8)
    x = rng.integers(0, 256, (1, 8, 8, 8), dtype=np.int64).astype(np.uint8)
    w = rng.integers(0, 256, (8, 3, 3, 8), dtype=np.int64).astype(np.uint8)
    b = rng.integers(-200, 200, 8, dtype=np.int64).astype(np.int32)
    outs = {}
    for legacy, pads in ((nw.LEGACY_TENSORFLOW_NHWC, (0, 1, 0, 1)), (nw.LEGACY_CAFFE_NHWC, (1, 1, 1, 1))):
        mb = nw.ModelBuilder(legacy)
        ti = mb.tensor((1, 8, 8, 8), "uint8", 0.02, 100)
        tw = mb.tensor(w.shape, "uint8", 0.005, 120, data=w)
        tb = mb.tensor((8,), "int32", 0.0001, 0, data=b)
        to = mb.tensor((1, 4, 4, 8), "uint8", 0.05, 128)
        mb.op("CONV_2D", [ti, tw, tb], [to], "Conv2DOptions", nw.Table(f0=("i8", nw.PAD_SAME), f1=("i32", 2), f2=("i32", 2), f3=("i8", 0)))
        mb.inputs, mb.outputs = [ti], [to]
        model = enn.Model(ctx, mb.finish())
        try:
            (y,) = model.execute([x])
        finally:
            model.close()
        pt, pb, pl, pr = pads
        d = enn.conv_desc(n=1, h=8, w=8, cin=8, cout=8, kh=3, kw=3, stride_h=2, stride_w=2, pad_t=pt, pad_b=pb, pad_l=pl, pad_r=pr, weight_layout=enn.W_OHWI,
                          in_scale=0.02, in_zp=100, w_scale=0.005, w_zp=120, bias_scale=0.0001, out_scale=0.05, out_zp=128)
        assert np.array_equal(y, orc.conv2d(d, x, w, b).reshape(-1)), legacy
        outs[legacy] = y
    assert not np.array_equal(outs[nw.LEGACY_TENSORFLOW_NHWC], outs[nw.LEGACY_CAFFE_NHWC])


@pytest.mark.gpu
def test_nnc_android_nn_transposed_convolution(orc, ctx):
    """ANDROID_NN model: explicit {l, r, t, b} padding values and an OHWI transposed-convolution filter."""
    rng = np.random.default_rng(9)
    x = rng.integers(0, 256, (2, 6, 5, 16), dtype=np.int64).astype(np.uint8)
    w = rng.integers(0, 256, (8, 4, 4, 16), dtype=np.int64).astype(np.uint8)
    b = rng.integers(-500, 500, 8, dtype=np.int64).astype(np.int32)
    mb = nw.ModelBuilder(nw.LEGACY_ANDROID_NN)
    ti = mb.tensor(x.shape, "uint8", 0.02, 128)
    tw = mb.tensor(w.shape, "uint8", 0.004, 120, data=w)
    tb = mb.tensor((8,), "int32", 0.02 * 0.004, 0, data=b)
    to = mb.tensor((2, 12, 10, 8), "uint8", 0.05, 128)
    mb.op("TRANSPOSE_CONV", [ti, tw, tb], [to], "TransposeConvOptions",
          nw.Table(f0=("i8", nw.PAD_SAME), f1=("i32", 2), f2=("i32", 2), f3=("i32", 1), f4=("i8", 0), f5=nw.Vec("i32", [1, 1, 1, 1])))
    mb.inputs, mb.outputs = [ti], [to]
    model = enn.Model(ctx, mb.finish())
    try:
        (y,) = model.execute([x])
    finally:
        model.close()
    d = enn.conv_desc(n=2, h=6, w=5, cin=16, cout=8, kh=4, kw=4, stride_h=2, stride_w=2, pad_t=1, pad_b=1, pad_l=1, pad_r=1, weight_layout=enn.W_OHWI,
                      in_scale=0.02, in_zp=128, w_scale=0.004, w_zp=120, bias_scale=float(np.float32(0.02) * np.float32(0.004)), out_scale=0.05, out_zp=128)
    assert np.array_equal(y, orc.deconv(d, x, w, b).reshape(-1))


@pytest.mark.gpu
def test_nnc_rejects_bad_files(ctx):
    with pytest.raises(enn.EnnError):
        enn.Model(ctx, b"\0" * 64)
    blob, _, _ = _graph_model(nw.LEGACY_TENSORFLOW_NHWC)
    with pytest.raises(enn.EnnError):
        enn.Model(ctx, blob[:len(blob) // 2])               # truncated: every access is bounds-checked
    mb = nw.ModelBuilder(4)                                  # TENSORFLOW_NCHW
    t = mb.tensor((1, 4, 4, 4), "uint8", 0.1, 0)
    mb.inputs, mb.outputs = [t], [t]
    with pytest.raises(enn.EnnError):
        enn.Model(ctx, mb.finish())
