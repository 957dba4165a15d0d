"""MobileNetV2-1.0 224x224 uint8-quantized graph built from the library's operators.

The reference ships no MobileNetV2-u8 model file and no calibration data, so the graph is synthetic:
random int8 per-channel weights, random per-channel scales, int32 biases, and per-layer activation scales
fixed by a calibration pass over a few seeded uniform images (exact integer arithmetic in float64 numpy).
The topology is the standard one: 3x3/s2 stem, 17 inverted-residual blocks (1x1 expand, 3x3 depthwise,
1x1 project, residual add where shapes allow), 1x1 to 1280, global average pool, FullyConnected to 1000.

`build_model` returns plain numpy data; `make_oplist` turns it into an operator list through the C ABI
(convolutions -> enn_b200_conv2d_prepare, depthwise -> enn_b200_depthwise_prepare, ...), one op per layer.
"""
import numpy as np

# (expansion t, output channels c, repeats n, first stride s)
BLOCKS = [(1, 16, 1, 1), (6, 24, 2, 2), (6, 32, 3, 2), (6, 64, 4, 2), (6, 96, 3, 1), (6, 160, 3, 2), (6, 320, 1, 1)]
ACT_NONE, ACT_RELU6 = 0, 3


def _same_pad(in_size, k, s):
    out = (in_size + s - 1) // s
    total = max(0, (out - 1) * s + k - in_size)
    return total // 2, (total + 1) // 2, out


def topology(resolution=224, num_classes=1000):
    """Layer list without weights: dicts with kind, geometry, input tensor names."""
    layers = []
    h = resolution
    pt, pb, oh = _same_pad(h, 3, 2)
    layers.append(dict(kind="conv", name="stem", src="input", h=h, cin=3, cout=32, k=3, stride=2, pad=(pt, pb), act=ACT_RELU6))
    h, c, prev = oh, 32, "stem"
    bi = 0
    for t, cout, n, s in BLOCKS:
        for i in range(n):
            stride = s if i == 0 else 1
            name = f"b{bi}"
            x_in = prev
            cur, cc = prev, c
            if t != 1:
                layers.append(dict(kind="conv", name=name + "_expand", src=cur, h=h, cin=cc, cout=cc * t, k=1, stride=1, pad=(0, 0), act=ACT_RELU6))
                cur, cc = name + "_expand", cc * t
            pt, pb, oh = _same_pad(h, 3, stride)
            layers.append(dict(kind="dw", name=name + "_dw", src=cur, h=h, cin=cc, cout=cc, k=3, stride=stride, pad=(pt, pb), act=ACT_RELU6))
            cur = name + "_dw"
            layers.append(dict(kind="conv", name=name + "_project", src=cur, h=oh, cin=cc, cout=cout, k=1, stride=1, pad=(0, 0), act=ACT_NONE))
            cur = name + "_project"
            if stride == 1 and c == cout:
                layers.append(dict(kind="add", name=name + "_add", src=x_in, src2=cur, h=oh, cin=cout, cout=cout))
                cur = name + "_add"
            h, c, prev = oh, cout, cur
            bi += 1
    layers.append(dict(kind="conv", name="head", src=prev, h=h, cin=c, cout=1280, k=1, stride=1, pad=(0, 0), act=ACT_RELU6))
    layers.append(dict(kind="pool", name="pool", src="head", h=h, cin=1280, cout=1280, k=h))
    layers.append(dict(kind="fc", name="fc", src="pool", h=1, cin=1280, cout=num_classes))
    return layers


def _conv_acc(x, w_ohwi, stride, pad, in_zp):
    """Integer conv accumulators in float64 (exact): x uint8 NHWC, w int8 [O][kh][kw][I]; zero-point padded."""
    n, h, _, cin = x.shape
    o, kh, kw, _ = w_ohwi.shape
    pt, pb = pad
    xp = np.full((n, h + pt + pb, h + pt + pb, cin), in_zp, np.float64)
    xp[:, pt:pt + h, pt:pt + h] = x
    xp -= in_zp
    oh = (h + pt + pb - kh) // stride + 1
    acc = np.zeros((n, oh, oh, o), np.float64)
    wf = w_ohwi.astype(np.float64)
    for ky in range(kh):
        for kx in range(kw):
            patch = xp[:, ky:ky + (oh - 1) * stride + 1:stride, kx:kx + (oh - 1) * stride + 1:stride]
            acc += patch.reshape(-1, cin) .dot(wf[:, ky, kx, :].T).reshape(n, oh, oh, o)
    return acc


def _dw_acc(x, w_o33, stride, pad, in_zp):
    n, h, _, c = x.shape
    pt, pb = pad
    xp = np.full((n, h + pt + pb, h + pt + pb, c), in_zp, np.float64)
    xp[:, pt:pt + h, pt:pt + h] = x
    xp -= in_zp
    oh = (h + pt + pb - 3) // stride + 1
    acc = np.zeros((n, oh, oh, c), np.float64)
    for ky in range(3):
        for kx in range(3):
            acc += xp[:, ky:ky + (oh - 1) * stride + 1:stride, kx:kx + (oh - 1) * stride + 1:stride] * w_o33[:, ky, kx].astype(np.float64)
    return acc


def _quantize_multiplier(m):
    if m == 0.0:
        return 0, 0
    q, e = np.frexp(m)
    qf = int(round(q * (1 << 31)))
    if qf == 1 << 31:
        qf //= 2
        e += 1
    return qf, int(e)


def _requant_np(acc, mult, shift, zp, lo, hi):
    """Vectorised restatement of the fixed-point tail, used only to propagate calibration images."""
    acc = acc.astype(np.int64)
    out = np.empty(acc.shape, np.int64)
    for c in range(acc.shape[-1]):
        m, s = int(mult[c]), int(shift[c])
        a = acc[..., c] << max(s, 0)
        x = (a * m + (1 << 30)) >> 31
        e = max(-s, 0)
        if e > 0:
            x = (x + (1 << (e - 1)) - (x < 0)) >> e
        out[..., c] = x
    return np.clip(out + zp, lo, hi).astype(np.uint8)


def build_model(seed=0, calib_images=2, resolution=224, num_classes=1000):
    """Random weights + calibrated activation scales.  Returns (layers, input_quant)."""
    rng = np.random.default_rng(seed)
    layers = topology(resolution, num_classes)
    in_scale, in_zp = np.float32(1.0 / 128.0), 128
    calib = rng.integers(0, 256, (calib_images, resolution, resolution, 3), dtype=np.int64).astype(np.uint8)
    acts = {"input": (calib, in_scale, in_zp)}
    for L in layers:
        x, xs, xz = acts[L["src"]]
        L["in_scale"], L["in_zp"] = np.float32(xs), int(xz)
        if L["kind"] in ("conv", "dw", "fc"):
            cout, cin, k = L["cout"], L["cin"], L.get("k", 1)
            if L["kind"] == "dw":
                w = rng.integers(-127, 128, (cout, 1, k, k), dtype=np.int64).astype(np.int8)          # [C][1][3][3]
            else:
                w = rng.integers(-127, 128, (cout, k, k, cin), dtype=np.int64).astype(np.int8)        # OHWI
            scales = np.exp(rng.uniform(np.log(2e-3), np.log(2e-2), cout)).astype(np.float32)
            bias = rng.integers(-1000, 1001, cout, dtype=np.int64).astype(np.int32)
            if L["kind"] == "dw":
                acc = _dw_acc(x, w[:, 0], L["stride"], L["pad"], xz)
            elif L["kind"] == "fc":
                acc = (x.reshape(x.shape[0], -1).astype(np.float64) - xz).dot(w.reshape(cout, cin).astype(np.float64).T)
                acc = acc.reshape(x.shape[0], 1, 1, cout)
            else:
                acc = _conv_acc(x, w, L["stride"], L["pad"], xz)
            acc = acc + bias
            real = acc * (np.float64(xs) * scales.astype(np.float64))
            if L.get("act", ACT_NONE) == ACT_RELU6:
                top = min(6.0, max(float(real.max()), 1e-3))
                out_scale, out_zp = np.float32(top / 255.0), 0
            else:
                top = max(float(np.abs(real).max()), 1e-3)
                out_scale, out_zp = np.float32(top / 127.0), 128
            L.update(w=w, scales=scales, bias=bias, out_scale=out_scale, out_zp=out_zp)
            mult, shift = zip(*[_quantize_multiplier(float(np.float64(xs) * np.float64(s) / np.float64(out_scale))) for s in scales])
            if L.get("act", ACT_NONE) == ACT_RELU6:
                lo = max(0, out_zp + int(np.round(np.float32(0.0) / out_scale)))
                hi = min(255, out_zp + int(np.round(np.float32(6.0) / out_scale)))
            else:
                lo, hi = 0, 255
            y = _requant_np(acc, mult, shift, out_zp, lo, hi)
            acts[L["name"]] = (y, out_scale, out_zp)
        elif L["kind"] == "add":
            a, sa, za = acts[L["src"]]
            b, sb, zb = acts[L["src2"]]
            real = (a.astype(np.float64) - za) * float(sa) + (b.astype(np.float64) - zb) * float(sb)
            top = max(float(np.abs(real).max()), 1e-3)
            out_scale, out_zp = np.float32(top / 127.0), 128
            L.update(in2_scale=np.float32(sb), in2_zp=int(zb), out_scale=out_scale, out_zp=out_zp)
            y = np.clip(np.round(real / float(out_scale)) + out_zp, 0, 255).astype(np.uint8)   # calibration only
            acts[L["name"]] = (y, out_scale, out_zp)
        elif L["kind"] == "pool":
            s = x.astype(np.int64).sum(axis=(1, 2), keepdims=True)
            n = x.shape[1] * x.shape[2]
            y = ((s + n // 2) // n).astype(np.uint8)
            L.update(out_scale=np.float32(xs), out_zp=int(xz))
            acts[L["name"]] = (y, xs, xz)
    return layers, (in_scale, in_zp)


def layer_descs(enn, L, batch):
    """The C-ABI descriptor of one layer for a given batch size."""
    if L["kind"] in ("conv", "dw"):
        pt, pb = L["pad"]
        return enn.conv_desc(n=batch, h=L["h"], w=L["h"], cin=L["cin"], cout=L["cout"], kh=L["k"], kw=L["k"],
                             stride_h=L["stride"], stride_w=L["stride"], pad_t=pt, pad_b=pb, pad_l=pt, pad_r=pb,
                             groups=1, activation=L["act"], act_dtype=enn.U8, weight_dtype=enn.S8,
                             weight_layout=enn.W_OIHW if L["kind"] == "dw" else enn.W_OHWI, per_channel=1,
                             in_scale=L["in_scale"], in_zp=L["in_zp"], out_scale=L["out_scale"], out_zp=L["out_zp"])
    if L["kind"] == "fc":
        return enn.FcDesc(m=batch, k=L["cin"], n=L["cout"], activation=0, act_dtype=enn.U8, weight_dtype=enn.S8,
                          per_channel=1, in_scale=L["in_scale"], in_zp=L["in_zp"], w_scale=1.0, w_zp=0, bias_scale=1.0,
                          out_scale=L["out_scale"], out_zp=L["out_zp"])
    if L["kind"] == "add":
        oh = L["h"]
        return enn.AddDesc(count=batch * oh * oh * L["cout"], activation=0, act_dtype=enn.U8, in0_scale=L["in_scale"],
                           in0_zp=L["in_zp"], in1_scale=L["in2_scale"], in1_zp=L["in2_zp"], out_scale=L["out_scale"],
                           out_zp=L["out_zp"])
    if L["kind"] == "pool":
        return enn.PoolDesc(n=batch, h=L["h"], w=L["h"], c=L["cin"], kh=L["k"], kw=L["k"], stride_h=1, stride_w=1,
                            pad_t=0, pad_l=0, out_h=1, out_w=1, activation=0, act_dtype=enn.U8,
                            out_scale=L["out_scale"], out_zp=L["out_zp"])
    raise ValueError(L["kind"])


def graph_work(layers, batch):
    """(multiply-accumulates, algorithmic bytes) of one pass over `batch` images, counted as the library counts them per
    operator: input + output + weights + 12 bytes of per-channel constants per output channel, each once."""
    macs = nbytes = 0
    for L in layers:
        h = L["h"]
        if L["kind"] in ("conv", "dw"):
            pt, pb = L["pad"]
            oh = (h + pt + pb - L["k"]) // L["stride"] + 1
            cin_g = 1 if L["kind"] == "dw" else L["cin"]
            macs += batch * oh * oh * L["cout"] * L["k"] * L["k"] * cin_g
            nbytes += batch * h * h * L["cin"] + batch * oh * oh * L["cout"] + L["k"] * L["k"] * cin_g * L["cout"] + 12 * L["cout"]
        elif L["kind"] == "fc":
            macs += batch * L["cin"] * L["cout"]
            nbytes += batch * L["cin"] + batch * L["cout"] + L["cin"] * L["cout"] + 12 * L["cout"]
        elif L["kind"] == "add":
            nbytes += 3 * batch * h * h * L["cout"]
        else:
            nbytes += batch * h * h * L["cin"] + batch * L["cin"]
    return macs, nbytes


def make_oplist(enn, ctx, layers, batch, resolution=224):
    """Prepares every layer through the C ABI and wires them into an operator list.
    Returns (oplist, info) where info carries per-layer work figures for reporting."""
    ol = enn.OpList(ctx)
    tid = {"input": ol.tensor(batch * resolution * resolution * 3)}
    per_layer = []
    for L in layers:
        d = layer_descs(enn, L, batch)
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
        i = op.info
        per_layer.append(dict(name=L["name"], kind=L["kind"], impl=i.impl, macs=i.macs, bytes=i.algorithmic_bytes,
                              out_bytes=i.out_bytes, launches=i.kernel_launches))
        tid[L["name"]] = ol.tensor(i.out_bytes)
        ins = [tid[L["src"]]] + ([tid[L["src2"]]] if L["kind"] == "add" else [])
        ol.add(op, ins, tid[L["name"]])
    out_bytes = batch * layers[-1]["cout"]
    ol.set_io([tid["input"]], [tid[layers[-1]["name"]]], [out_bytes])
    ol.finalize()
    info = dict(per_layer=per_layer, macs=sum(p["macs"] for p in per_layer), bytes=sum(p["bytes"] for p in per_layer),
                launches=sum(p["launches"] for p in per_layer), tensor_ids=tid)
    return ol, info
